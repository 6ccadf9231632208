// The small kernels around blocks whose sub-layers join the residual stream through a learned gate, around a layer
// norm that takes the mean out, and around mixers that stand side by side.  Every sum, norm and gate is float in
// both builds; act_t is only what the projections hand in and what the next projection reads.
//
//   gated add + layer norm   x <- x + sigmoid(p + b) * delta (float, in place), then (x - mean) / sqrt(var + eps) * w
//                            as act_t; the gate, the delta or both may be absent; a choice of rows reads only
//   gated rows               delta * sigmoid(p + b) as act_t, for a norm of another kind that follows such a block
//   bias                     rows += b
//   scaled sum               a x + b y
//   mixed queries            q~[h, c, :] = sum over the heads g of key/value group c of T[h, g] q[g, :]
#include "common.cuh"

__device__ __forceinline__ float gb_sigmoid(float z) { return 1.0f / (1.0f + expf(-z)); }

// One block per output row.  The row stays in shared memory between the three passes (sum, squared deviations,
// output), so the variance is the mean of the squared deviations from the mean itself, not a difference of sums.
__global__ void gated_add_layer_norm_kernel(float* __restrict__ residual, const act_t* __restrict__ delta,
                                            const act_t* __restrict__ gate_pre, const float* __restrict__ gate_bias,
                                            const float* __restrict__ weight, float eps, act_t* __restrict__ out,
                                            const int* __restrict__ rows, int width) {
    extern __shared__ float row_s[];
    __shared__ float red[32];
    ib_grid_dependency_sync();
    const long r = rows ? rows[blockIdx.x] : blockIdx.x;
    float* res = residual + r * width;
    float sum = 0.0f;
    for (int j = threadIdx.x; j < width; j += blockDim.x) {
        float v = res[j];
        if (delta) {
            float d = ib_to_float(delta[r * width + j]);
            if (gate_pre) d *= gb_sigmoid(ib_to_float(gate_pre[r * width + j]) + (gate_bias ? gate_bias[j] : 0.0f));
            v += d;
            if (!rows) res[j] = v;
        }
        row_s[j] = v;
        sum += v;
    }
    const float mean = ib_block_sum(sum, red) / (float)width;
    float ss = 0.0f;
    for (int j = threadIdx.x; j < width; j += blockDim.x) {
        const float c = row_s[j] - mean;
        ss += c * c;
    }
    const float inv = 1.0f / sqrtf(ib_block_sum(ss, red) / (float)width + eps);
    act_t* dst = out + (long)blockIdx.x * width;
    for (int j = threadIdx.x; j < width; j += blockDim.x)
        dst[j] = ib_from_float<act_t>((row_s[j] - mean) * inv * weight[j]);
}

// residual float [n, width] (updated in place unless `rows` chooses); delta, gate_pre act_t [n, width] or absent;
// gate_bias float [width] or absent; out act_t [n_out, width].
IB_EXPORT int ib_gated_add_layer_norm(float* residual, const void* delta, const void* gate_pre, const float* gate_bias,
                                      const float* weight, float eps, void* out, const int* rows, int n_out, int width,
                                      cudaStream_t stream) {
    if (n_out <= 0) return IB_OK;
    if (width <= 0 || residual == nullptr || weight == nullptr || out == nullptr || (gate_pre && !delta))
        return IB_ERR_ARGUMENT;
    if (width > 11 * 1024) return IB_ERR_UNSUPPORTED;      // the row in 44 KB of shared memory
    const int threads = width >= 2048 ? 512 : (width >= 512 ? 256 : 128);
    ib_launch(gated_add_layer_norm_kernel, n_out, threads, (size_t)width * sizeof(float), stream, residual,
              (const act_t*)delta, (const act_t*)gate_pre, gate_bias, weight, eps, (act_t*)out, rows, width);
    return ib_launch_status();
}

__global__ void gated_rows_kernel(const act_t* __restrict__ delta, const act_t* __restrict__ gate_pre,
                                  const float* __restrict__ gate_bias, act_t* __restrict__ out, int width, long total) {
    ib_grid_dependency_sync();
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
        const int j = (int)(i % width);
        const float g = gb_sigmoid(ib_to_float(gate_pre[i]) + (gate_bias ? gate_bias[j] : 0.0f));
        out[i] = ib_from_float<act_t>(ib_to_float(delta[i]) * g);
    }
}

IB_EXPORT int ib_gated_rows(const void* delta, const void* gate_pre, const float* gate_bias, void* out, int n_rows,
                            int width, cudaStream_t stream) {
    if (n_rows <= 0) return IB_OK;
    if (width <= 0 || delta == nullptr || gate_pre == nullptr || out == nullptr) return IB_ERR_ARGUMENT;
    const long total = (long)n_rows * width;
    long blocks = (total + 255) / 256;
    if (blocks > 148L * 16) blocks = 148L * 16;
    ib_launch(gated_rows_kernel, (int)blocks, 256, 0, stream, (const act_t*)delta, (const act_t*)gate_pre, gate_bias,
              (act_t*)out, width, total);
    return ib_launch_status();
}

__global__ void bias_add_kernel(act_t* __restrict__ x, long ld, const float* __restrict__ bias, int width) {
    ib_grid_dependency_sync();
    const int j = blockIdx.x * blockDim.x + threadIdx.x;
    if (j >= width) return;
    act_t* p = x + (long)blockIdx.y * ld + j;
    *p = ib_from_float<act_t>(ib_to_float(*p) + bias[j]);
}

// x act_t [n_rows, ld]: the first `width` columns of every row get bias [width] added.
IB_EXPORT int ib_bias_add(void* x, long ld, const float* bias, int n_rows, int width, cudaStream_t stream) {
    if (n_rows <= 0) return IB_OK;
    if (width <= 0 || ld < width || x == nullptr || bias == nullptr) return IB_ERR_ARGUMENT;
    for (int r0 = 0; r0 < n_rows; r0 += 65535) {
        const int rows = n_rows - r0 < 65535 ? n_rows - r0 : 65535;
        ib_launch(bias_add_kernel, dim3((width + 255) / 256, rows), 256, 0, stream, (act_t*)x + (long)r0 * ld, ld, bias,
                  width);
    }
    return ib_launch_status();
}

__global__ void scaled_sum_kernel(const act_t* __restrict__ x, float a, const act_t* __restrict__ y, float b,
                                  act_t* __restrict__ out, long total) {
    ib_grid_dependency_sync();
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x)
        out[i] = ib_from_float<act_t>(a * ib_to_float(x[i]) + b * ib_to_float(y[i]));
}

IB_EXPORT int ib_scaled_sum(const void* x, float a, const void* y, float b, void* out, long total, cudaStream_t stream) {
    if (total <= 0) return IB_OK;
    if (x == nullptr || y == nullptr || out == nullptr) return IB_ERR_ARGUMENT;
    long blocks = (total + 255) / 256;
    if (blocks > 148L * 16) blocks = 148L * 16;
    ib_launch(scaled_sum_kernel, (int)blocks, 256, 0, stream, (const act_t*)x, a, (const act_t*)y, b, (act_t*)out,
              total);
    return ib_launch_status();
}

// q act_t [n, H, D] -> out act_t [n, H, G * D]: out[r, h, c * D + e] = sum over g in group c of mix[h, g] q[r, g, e]
// (mix float [H, H]; group c holds the heads c * (H / G) .. (c + 1) * (H / G) - 1).  A score of head h against the
// keys of all groups side by side is then the mix of the heads' own scores: the mixing of scores across heads is
// linear, so it can be done on the queries once per token instead of on every (query, key) pair.
__global__ void mix_queries_kernel(const act_t* __restrict__ q, const float* __restrict__ mix, act_t* __restrict__ out,
                                   int H, int G, int D) {
    ib_grid_dependency_sync();
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    const int per_head = G * D;
    if (idx >= H * per_head) return;
    const long r = blockIdx.y;
    const int h = idx / per_head, rest = idx - h * per_head, c = rest / D, e = rest - c * D;
    const int per_group = H / G;
    const act_t* src = q + (r * H + (long)c * per_group) * D + e;
    float acc = 0.0f;
    for (int i = 0; i < per_group; ++i) acc = fmaf(mix[h * H + c * per_group + i], ib_to_float(src[(long)i * D]), acc);
    out[r * H * per_head + idx] = ib_from_float<act_t>(acc);
}

IB_EXPORT int ib_mix_queries(const void* q, const float* mix, void* out, int n_rows, int H, int G, int D,
                             cudaStream_t stream) {
    if (n_rows <= 0) return IB_OK;
    if (H <= 0 || G <= 0 || H % G || D <= 0 || q == nullptr || mix == nullptr || out == nullptr) return IB_ERR_ARGUMENT;
    const int total = H * G * D;
    for (int r0 = 0; r0 < n_rows; r0 += 65535) {
        const int rows = n_rows - r0 < 65535 ? n_rows - r0 : 65535;
        ib_launch(mix_queries_kernel, dim3((total + 255) / 256, rows), 256, 0, stream,
                  (const act_t*)q + (long)r0 * H * D, mix, (act_t*)out + (long)r0 * total, H, G, D);
    }
    return ib_launch_status();
}
