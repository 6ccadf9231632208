// The small kernels around blocks that norm after the sum and around mixers with a scalar decay per head
// (a fixed-decay linear attention, a state-space mixer with a short convolution), and a feed-forward of routed
// experts.  Every sum, norm, gate, decay and angle is float in both builds; act_t is only what the projections
// hand in and what the next projection reads.
//
//   norm after the sum      x <- norm(alpha x + delta) * w, the stream itself normalised, with a copy as act_t
//   heads to float          slices of a projection's rows as float, rotated by position and scaled where asked
//   convolution and gates   silu(causal convolution + bias) per channel over a request's rows and the inputs that
//                           its state keeps, and per head dt = softplus(p + b), keep = exp(-exp(A) dt), take = dt
//   convolution state       the last taps - 1 inputs of every request, after the step
//   gate, then norm         (y * silu(z)) divided by the root mean square of each of `groups` parts, times w
//   clamped gate            min(g, c) * sigmoid(s min(g, c)) * (clamp(u, -c, c) + 1)
//   router                  top-k of logits + bias, softmax over the chosen, as a dense row of weights
//   routed gate             silu(g) * u * weight of the column's expert
#include "common.cuh"

__device__ __forceinline__ float sm_silu(float z) { return z / (1.0f + expf(-z)); }
__device__ __forceinline__ float sm_sigmoid(float z) { return 1.0f / (1.0f + expf(-z)); }
__device__ __forceinline__ float sm_softplus(float z) { return z > 20.0f ? z : log1pf(expf(z)); }
// the tanh form of gelu: 0.5 z (1 + tanh(sqrt(2 / pi) (z + 0.044715 z^3)))
__device__ __forceinline__ float sm_gelu_tanh(float z) {
    return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}
// What a gated feed-forward makes of a gate g and an up value u.  mode 0: g' sigmoid(slope g') (u' + 1) with
// g' = min(g, limit), u' = clamp(u, -limit, limit); mode 1: gelu_tanh(g) u; mode 2: silu(g) u.
__device__ __forceinline__ float sm_gate_value(int mode, float g, float u, float limit, float slope) {
    if (mode == 1) return sm_gelu_tanh(g) * u;
    if (mode == 2) return sm_silu(g) * u;
    g = fminf(g, limit);
    u = fminf(fmaxf(u, -limit), limit);
    return g * sm_sigmoid(slope * g) * (u + 1.0f);
}

// ---------------------------------------------------------------------------
// residual[r, :] <- (alpha * residual[r, :] + delta[r, :]) / rms * weight   (in place, float)
// copy[r, :] = the same as act_t (what the next sub-layer reads; may be absent).  delta may be absent.
// ---------------------------------------------------------------------------
__global__ void scaled_add_norm_kernel(float* __restrict__ residual, const act_t* __restrict__ delta, float alpha,
                                       const float* __restrict__ weight, float eps, act_t* __restrict__ copy,
                                       int width) {
    __shared__ float red[32];
    ib_grid_dependency_sync();
    const size_t base = (size_t)blockIdx.x * width;
    float ss = 0.0f;
    for (int j = threadIdx.x; j < width; j += blockDim.x) {
        float v = alpha * residual[base + j];
        if (delta) v += ib_to_float(delta[base + j]);
        residual[base + j] = v;          // read again below by the thread that wrote it
        ss += v * v;
    }
    ss = ib_block_sum(ss, red);
    const float inv = 1.0f / sqrtf(ss / (float)width + eps);
    for (int j = threadIdx.x; j < width; j += blockDim.x) {
        const float v = residual[base + j] * inv * weight[j];
        residual[base + j] = v;
        if (copy) copy[base + j] = ib_from_float<act_t>(v);
    }
}

// Four elements per thread and step, the row kept in registers between the two passes: for widths that are
// multiples of 4 and at most 4 * SAN_KEEP * (threads per block).
#define SAN_KEEP 4
struct alignas(sizeof(act_t) * 4) SanActVec4 { act_t v[4]; };

__global__ void scaled_add_norm_vec4_kernel(float* __restrict__ residual, const act_t* __restrict__ delta, float alpha,
                                            const float* __restrict__ weight, float eps, act_t* __restrict__ copy,
                                            int width) {
    __shared__ float red[32];
    ib_grid_dependency_launch();
    const int n4 = width >> 2;
    float4 wk[SAN_KEEP];       // the norm's weights are fetched while the kernel before this one still runs
#pragma unroll
    for (int k = 0; k < SAN_KEEP; ++k) {
        const int j = threadIdx.x + k * blockDim.x;
        if (j < n4) wk[k] = reinterpret_cast<const float4*>(weight)[j];
    }
    ib_grid_dependency_wait();
    float4* res = reinterpret_cast<float4*>(residual + (size_t)blockIdx.x * width);
    const SanActVec4* del = delta ? reinterpret_cast<const SanActVec4*>(delta + (size_t)blockIdx.x * width) : nullptr;
    float4 keep[SAN_KEEP];
    float ss = 0.0f;
#pragma unroll
    for (int k = 0; k < SAN_KEEP; ++k) {
        const int j = threadIdx.x + k * blockDim.x;
        if (j < n4) {
            float4 v = res[j];
            v.x *= alpha; v.y *= alpha; v.z *= alpha; v.w *= alpha;
            if (del) {
                const SanActVec4 d = del[j];
                v.x += ib_to_float(d.v[0]); v.y += ib_to_float(d.v[1]);
                v.z += ib_to_float(d.v[2]); v.w += ib_to_float(d.v[3]);
            }
            ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
            keep[k] = v;
        }
    }
    ss = ib_block_sum(ss, red);
    const float inv = 1.0f / sqrtf(ss / (float)width + eps);
    SanActVec4* dst = copy ? reinterpret_cast<SanActVec4*>(copy + (size_t)blockIdx.x * width) : nullptr;
#pragma unroll
    for (int k = 0; k < SAN_KEEP; ++k) {
        const int j = threadIdx.x + k * blockDim.x;
        if (j >= n4) break;
        float4 v = keep[k];
        v.x = v.x * inv * wk[k].x; v.y = v.y * inv * wk[k].y; v.z = v.z * inv * wk[k].z; v.w = v.w * inv * wk[k].w;
        res[j] = v;
        if (dst) {
            SanActVec4 o;
            o.v[0] = ib_from_float<act_t>(v.x); o.v[1] = ib_from_float<act_t>(v.y);
            o.v[2] = ib_from_float<act_t>(v.z); o.v[3] = ib_from_float<act_t>(v.w);
            dst[j] = o;
        }
    }
}

static inline bool sm_aligned16(const void* p) { return p == nullptr || ((uintptr_t)p & 15) == 0; }

IB_EXPORT int ib_scaled_add_norm(float* residual, const void* delta, float alpha, const float* weight, float eps,
                                 void* copy, int n_rows, int width, cudaStream_t stream) {
    if (n_rows <= 0) return IB_OK;
    if (width <= 0 || residual == nullptr || weight == nullptr) return IB_ERR_ARGUMENT;
    if ((width & 3) == 0 && width <= 4 * SAN_KEEP * 1024 && sm_aligned16(residual) && sm_aligned16(delta) &&
        sm_aligned16(weight) && sm_aligned16(copy)) {
        int t4 = 64;   // enough threads that SAN_KEEP float4 per thread hold the row
        while (4 * SAN_KEEP * t4 < width) t4 <<= 1;
        if (width >= 1024 && 4 * t4 < width && t4 < 256) t4 = 256;
        ib_launch(scaled_add_norm_vec4_kernel, n_rows, t4, 0, stream, residual, (const act_t*)delta, alpha, weight, eps,
                  (act_t*)copy, width);
        return ib_launch_status();
    }
    const int threads = width >= 2048 ? 512 : (width >= 512 ? 256 : 128);
    ib_launch(scaled_add_norm_kernel, n_rows, threads, 0, stream, residual, (const act_t*)delta, alpha, weight, eps,
              (act_t*)copy, width);
    return ib_launch_status();
}

// ---------------------------------------------------------------------------
// Up to three slices of a projection's rows as float: slice s is n_heads[s] heads of dim[s] numbers from column
// src_col[s] on, written from column dst_col[s] of the float rows; where rotate[s] is set the first rot_dim of
// each head turn by the row's position (element i with i + rot_dim / 2; tables [positions, rot_dim / 2]); every
// number is multiplied by scale[s]; where silu[s] is set the number goes through silu first (a slice is rotated or
// goes through silu, not both).
// ---------------------------------------------------------------------------
struct HeadSlices {
    int n, src_col[3], dst_col[3], n_heads[3], dim[3], rotate[3], silu[3];
    float scale[3];
};

__global__ void heads_to_float_kernel(const act_t* __restrict__ src, long ld, HeadSlices P, float* __restrict__ dst,
                                      long dst_ld, const float* __restrict__ cos_table,
                                      const float* __restrict__ sin_table, int rot_dim, int table_rows,
                                      const int* __restrict__ positions) {
    ib_grid_dependency_sync();
    const int row = blockIdx.y;
    int idx = blockIdx.x * blockDim.x + threadIdx.x;     // a number of the row's slices, counted through all of them
    int s = 0;
    while (s < P.n && idx >= P.n_heads[s] * P.dim[s]) { idx -= P.n_heads[s] * P.dim[s]; ++s; }
    if (s >= P.n) return;
    const act_t* in = src + (long)row * ld;
    const int half = rot_dim / 2;
    const int d = P.dim[s];
    const int j = idx % d;
    const act_t* h = in + P.src_col[s] + (idx - j);
    float v = ib_to_float(h[j]);
    if (P.rotate[s] && j < rot_dim) {
        int pos = positions[row];
        if (pos < 0) pos = 0;
        if (pos >= table_rows) pos = table_rows - 1;     // the host sizes the tables for every position of the model
        const int i = j < half ? j : j - half;
        const float c = cos_table[(long)pos * half + i], sn = sin_table[(long)pos * half + i];
        v = j < half ? v * c - ib_to_float(h[j + half]) * sn : v * c + ib_to_float(h[j - half]) * sn;
    }
    if (P.silu[s]) v = sm_silu(v);
    dst[(long)row * dst_ld + P.dst_col[s] + idx] = v * P.scale[s];
}

// The same for slices that do not turn, four numbers per thread: every slice's size, first column and row length
// is a multiple of four and both tensors start on a boundary of four of their numbers (the host checks).
__global__ void heads_to_float4_kernel(const act_t* __restrict__ src, long ld, HeadSlices P, float* __restrict__ dst,
                                       long dst_ld) {
    ib_grid_dependency_sync();
    struct alignas(4 * sizeof(act_t)) In4 { act_t v[4]; };
    const int row = blockIdx.y;
    int idx = (blockIdx.x * blockDim.x + threadIdx.x) * 4;
    int s = 0;
    while (s < P.n && idx >= P.n_heads[s] * P.dim[s]) { idx -= P.n_heads[s] * P.dim[s]; ++s; }
    if (s >= P.n) return;
    const In4 in = *reinterpret_cast<const In4*>(src + (long)row * ld + P.src_col[s] + idx);
    float v[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        v[i] = ib_to_float(in.v[i]);
        if (P.silu[s]) v[i] = sm_silu(v[i]);
        v[i] *= P.scale[s];
    }
    *reinterpret_cast<float4*>(dst + (long)row * dst_ld + P.dst_col[s] + idx) = make_float4(v[0], v[1], v[2], v[3]);
}

IB_EXPORT int ib_heads_to_float(const void* src, long ld, int n_slices, const int* src_col, const int* dst_col,
                                const int* n_heads, const int* dim, const int* rotate, const int* silu,
                                const float* scale, float* dst,
                                long dst_ld, const float* cos_table, const float* sin_table, int rot_dim, int table_rows,
                                const int* positions, int n_rows, cudaStream_t stream) {
    if (n_rows <= 0) return IB_OK;
    if (n_slices < 1 || n_slices > 3 || src == nullptr || dst == nullptr || rot_dim < 0 || (rot_dim & 1))
        return IB_ERR_ARGUMENT;
    HeadSlices P;
    P.n = n_slices;
    int total = 0;
    for (int s = 0; s < n_slices; ++s) {
        P.src_col[s] = src_col[s]; P.dst_col[s] = dst_col[s]; P.n_heads[s] = n_heads[s]; P.dim[s] = dim[s];
        P.rotate[s] = rotate[s]; P.scale[s] = scale[s]; P.silu[s] = silu ? silu[s] : 0;
        if (n_heads[s] <= 0 || dim[s] <= 0 || (rotate[s] && rot_dim > dim[s]) || (rotate[s] && P.silu[s]))
            return IB_ERR_ARGUMENT;
        if (rotate[s] && rot_dim > 0 && (cos_table == nullptr || sin_table == nullptr || positions == nullptr ||
                                        table_rows <= 0))
            return IB_ERR_ARGUMENT;
        total += n_heads[s] * dim[s];
    }
    if (n_rows > 65535) return IB_ERR_UNSUPPORTED;
    const int threads = 256;
    bool by_four = (ld % 4) == 0 && (dst_ld % 4) == 0 && ((uintptr_t)src % (4 * sizeof(act_t))) == 0 &&
                   ((uintptr_t)dst % 16) == 0;
    for (int s = 0; s < n_slices; ++s)
        by_four = by_four && !(rotate[s] && rot_dim > 0) && (dim[s] % 4) == 0 && (src_col[s] % 4) == 0 &&
                  (dst_col[s] % 4) == 0;
    if (by_four) {
        ib_launch(heads_to_float4_kernel, dim3((total / 4 + threads - 1) / threads, n_rows), threads, 0, stream,
                  (const act_t*)src, ld, P, dst, dst_ld);
        return ib_launch_status();
    }
    ib_launch(heads_to_float_kernel, dim3((total + threads - 1) / threads, n_rows), threads, 0, stream,
              (const act_t*)src, ld, P, dst, dst_ld, cos_table, sin_table, rot_dim, table_rows, positions);
    return ib_launch_status();
}

// ---------------------------------------------------------------------------
// Channel c < C of row r:  out[r, c] = silu(bias[c] + sum_j w[c, j] * input(r - (taps - 1 - j), c))  (bias may be absent),
// where input(t, c) is the projection's column conv_col + c of row t if t is a row of the same request in this
// step, and else what the request's state keeps: its last taps - 1 inputs, oldest first, [taps - 1, C] floats at
// conv_state_off of its slot (zeros for a new request: nothing stands before the start).
// Head h of row r (threads C .. C + H - 1):  dt = softplus(proj[r, dt_col + h] + dt_bias[h]),
// gates[r, h] = exp(-exp(a_log[h]) dt)  (what the state keeps),  gates[r, H + h] = dt  (what the input is taken by);
// with beta_col >= 0 the second is sigmoid(proj[r, beta_col + h]) instead (the step size of a delta rule).
// ---------------------------------------------------------------------------
__global__ void conv_silu_gates_kernel(const act_t* __restrict__ proj, long ld, int conv_col, int C, int taps,
                                       const float* __restrict__ w, const float* __restrict__ bias,
                                       const float* __restrict__ state, long slot_stride, long conv_state_off,
                                       const int* __restrict__ q_start, const int* __restrict__ slots,
                                       const int* __restrict__ row_request, float* __restrict__ out, int dt_col, int H,
                                       const float* __restrict__ dt_bias, const float* __restrict__ a_log,
                                       float* __restrict__ gates, int beta_col) {
    ib_grid_dependency_sync();
    const int row = blockIdx.y;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= C + H) return;
    const act_t* in = proj + (long)row * ld;
    if (c >= C) {
        const int h = c - C;
        const float dt = sm_softplus(ib_to_float(in[dt_col + h]) + dt_bias[h]);
        gates[(long)row * 2 * H + h] = expf(-expf(a_log[h]) * dt);
        gates[(long)row * 2 * H + H + h] = beta_col >= 0 ? sm_sigmoid(ib_to_float(in[beta_col + h])) : dt;
        return;
    }
    const int req = row_request[row];
    const int row0 = q_start[req];
    const float* kept = state + (long)slots[req] * slot_stride + conv_state_off;
    float acc = bias ? bias[c] : 0.0f;
    for (int j = 0; j < taps; ++j) {
        const int t = row - (taps - 1 - j);
        float v;
        if (t >= row0) v = ib_to_float(proj[(long)t * ld + conv_col + c]);
        else v = kept[(long)(taps - 1 - (row0 - t)) * C + c];
        acc = fmaf(w[(long)c * taps + j], v, acc);
    }
    out[(long)row * C + c] = sm_silu(acc);
}

IB_EXPORT int ib_conv_silu_gates(const void* proj, long ld, int conv_col, int C, int taps, const float* w,
                                 const float* bias, const float* state, long slot_stride, long conv_state_off,
                                 const int* q_start, const int* slots, const int* row_request, float* out, int dt_col,
                                 int H, const float* dt_bias, const float* a_log, float* gates, int beta_col,
                                 int n_rows, cudaStream_t stream) {
    if (n_rows <= 0) return IB_OK;
    if (C <= 0 || taps <= 0 || H <= 0 || proj == nullptr || w == nullptr || state == nullptr ||
        out == nullptr || gates == nullptr || dt_bias == nullptr || a_log == nullptr ||
        slot_stride < conv_state_off + (long)(taps - 1) * C)
        return IB_ERR_ARGUMENT;
    if (n_rows > 65535) return IB_ERR_UNSUPPORTED;
    const int threads = 128;
    ib_launch(conv_silu_gates_kernel, dim3((C + H + threads - 1) / threads, n_rows), threads, 0, stream,
              (const act_t*)proj, ld, conv_col, C, taps, w, bias, state, slot_stride, conv_state_off, q_start, slots,
              row_request, out, dt_col, H, dt_bias, a_log, gates, beta_col);
    return ib_launch_status();
}

// After the step: every request's state keeps its last taps - 1 inputs, oldest first.  A request that brought
// fewer rows than that keeps the youngest of what it held before them.  One thread per (request, channel) writes
// place k after it has read everything it needs from places above k.
__global__ void conv_state_shift_kernel(const act_t* __restrict__ proj, long ld, int conv_col, int C, int taps,
                                        float* __restrict__ state, long slot_stride, long conv_state_off,
                                        const int* __restrict__ q_start, const int* __restrict__ slots) {
    ib_grid_dependency_sync();
    const int req = blockIdx.y;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= C) return;
    const int row0 = q_start[req], n = q_start[req + 1] - row0;
    if (n <= 0) return;
    float* kept = state + (long)slots[req] * slot_stride + conv_state_off;
    for (int k = 0; k < taps - 1; ++k) {
        const int idx = n - (taps - 1) + k;      // which of the step's rows belongs at place k
        kept[(long)k * C + c] = idx >= 0 ? ib_to_float(proj[(long)(row0 + idx) * ld + conv_col + c])
                                         : kept[(long)(k + n) * C + c];
    }
}

IB_EXPORT int ib_conv_state_shift(const void* proj, long ld, int conv_col, int C, int taps, float* state,
                                  long slot_stride, long conv_state_off, const int* q_start, const int* slots,
                                  int n_requests, cudaStream_t stream) {
    if (n_requests <= 0 || taps <= 1) return IB_OK;
    if (C <= 0 || proj == nullptr || state == nullptr || n_requests > 65535) return IB_ERR_ARGUMENT;
    const int threads = 128;
    ib_launch(conv_state_shift_kernel, dim3((C + threads - 1) / threads, n_requests), threads, 0, stream,
              (const act_t*)proj, ld, conv_col, C, taps, state, slot_stride, conv_state_off, q_start, slots);
    return ib_launch_status();
}

// ---------------------------------------------------------------------------
// out[r, :] = norm_in_groups(y[r, :] * silu(z[r, :])) * weight (gated first, normed second); each of `groups`
// equal consecutive parts of the row is divided by its own root mean square.  One warp per part.
// ---------------------------------------------------------------------------
__global__ void gate_group_norm_kernel(const float* __restrict__ y, const act_t* __restrict__ z, long z_ld,
                                       const float* __restrict__ weight, int groups, int part, float eps,
                                       act_t* __restrict__ out, int warps_per_part) {
    __shared__ float sums[32];
    ib_grid_dependency_sync();
    const int row = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
    const long inner = (long)groups * part;
    // few parts: every part has `warps_per_part` warps of the block (one round); many parts: a warp each, in rounds
    const int parts_per_round = n_warps / warps_per_part;
    const int sub = warp % warps_per_part, lanes = 32 * warps_per_part;
    for (int g0 = 0; g0 < groups; g0 += parts_per_round) {
        const int g = g0 + warp / warps_per_part;
        const bool mine = g < groups && warp / warps_per_part < parts_per_round;
        const float* yr = y + (long)row * inner + (long)g * part;
        const act_t* zr = z + (long)row * z_ld + (long)g * part;
        float ss = 0.0f;
        if (mine)
            for (int j = sub * 32 + lane; j < part; j += lanes) {
                const float v = yr[j] * sm_silu(ib_to_float(zr[j]));
                ss += v * v;
            }
        ss = ib_warp_sum(ss);
        __syncthreads();                     // `sums` may still be read from the round before
        if (lane == 0) sums[warp] = ss;
        __syncthreads();
        if (!mine) continue;
        float total = 0.0f;
        for (int w = 0; w < warps_per_part; ++w) total += sums[(warp / warps_per_part) * warps_per_part + w];
        const float inv = 1.0f / sqrtf(total / (float)part + eps);
        for (int j = sub * 32 + lane; j < part; j += lanes) {
            const float v = yr[j] * sm_silu(ib_to_float(zr[j]));
            out[(long)row * inner + (long)g * part + j] = ib_from_float<act_t>(v * inv * weight[(long)g * part + j]);
        }
    }
}

IB_EXPORT int ib_gate_group_norm(const float* y, const void* z, long z_ld, const float* weight, int groups, int inner,
                                 float eps, void* out, int n_rows, cudaStream_t stream) {
    if (n_rows <= 0) return IB_OK;
    if (groups <= 0 || inner <= 0 || inner % groups || y == nullptr || z == nullptr || weight == nullptr)
        return IB_ERR_ARGUMENT;
    const int part = inner / groups;
    int warps = 8;
    while (warps > 1 && warps * 32 > inner) warps >>= 1;          // a narrow row needs no eight warps
    int per_part = warps / groups;                                 // warps that share one part
    if (per_part < 1) per_part = 1;
    while (per_part > 1 && per_part * 32 > part) per_part >>= 1;
    ib_launch(gate_group_norm_kernel, n_rows, 32 * warps, 0, stream, y, (const act_t*)z, z_ld, weight, groups, part, eps,
              (act_t*)out, per_part);
    return ib_launch_status();
}

// ---------------------------------------------------------------------------
// out[r, j] = g' * sigmoid(slope * g') * (u' + 1),  g' = min(gate_up[r, j], limit),
// u' = clamp(gate_up[r, inner + j], -limit, limit)
// ---------------------------------------------------------------------------
__global__ void clamped_gate_kernel(const act_t* __restrict__ gate_up, act_t* __restrict__ out, int inner, long total,
                                    float limit, float slope, int mode) {
    ib_grid_dependency_sync();
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
        const long r = i / inner;
        const int j = (int)(i - r * inner);
        out[i] = ib_from_float<act_t>(sm_gate_value(mode, ib_to_float(gate_up[r * 2 * inner + j]),
                                                    ib_to_float(gate_up[r * 2 * inner + inner + j]), limit, slope));
    }
}

// Sixteen bytes per thread (eight bfloat16 or four float) and one row per blockIdx.y, so that no thread divides to
// find its row: for inner sizes that are multiples of that many elements.
#define SM_VEC (16 / (int)sizeof(act_t))
struct alignas(16) SmActVec { act_t v[SM_VEC]; };

__global__ void clamped_gate_vec_kernel(const act_t* __restrict__ gate_up, act_t* __restrict__ out, int inner,
                                        float limit, float slope, int mode) {
    ib_grid_dependency_sync();
    const int j = blockIdx.x * blockDim.x + threadIdx.x;
    if (j >= inner / SM_VEC) return;
    const long r = blockIdx.y;
    const SmActVec g = reinterpret_cast<const SmActVec*>(gate_up + r * 2 * inner)[j];
    const SmActVec u = reinterpret_cast<const SmActVec*>(gate_up + r * 2 * inner + inner)[j];
    SmActVec o;
#pragma unroll
    for (int k = 0; k < SM_VEC; ++k)
        o.v[k] = ib_from_float<act_t>(sm_gate_value(mode, ib_to_float(g.v[k]), ib_to_float(u.v[k]), limit, slope));
    reinterpret_cast<SmActVec*>(out + r * inner)[j] = o;
}

// mode 0: the clamped form (limit > 0); mode 1: gelu_tanh(gate) * up (limit and slope are not read).
IB_EXPORT int ib_clamped_gate(const void* gate_up, void* out, int n_rows, int inner, float limit, float slope,
                              int mode, cudaStream_t stream) {
    if (n_rows <= 0) return IB_OK;
    if (inner <= 0 || mode < 0 || mode > 1 || (mode == 0 && !(limit > 0.0f))) return IB_ERR_ARGUMENT;
    if (inner % SM_VEC == 0 && sm_aligned16(gate_up) && sm_aligned16(out)) {
        const int nv = inner / SM_VEC;
        const int threads = nv >= 256 ? 256 : ((nv + 31) / 32) * 32;
        for (int r0 = 0; r0 < n_rows; r0 += 65535) {   // blockIdx.y holds at most 65,535 rows
            const int rows = n_rows - r0 < 65535 ? n_rows - r0 : 65535;
            ib_launch(clamped_gate_vec_kernel, dim3((nv + threads - 1) / threads, rows), threads, 0, stream,
                      (const act_t*)gate_up + (long)r0 * 2 * inner, (act_t*)out + (long)r0 * inner, inner, limit, slope,
                      mode);
        }
        return ib_launch_status();
    }
    const long total = (long)n_rows * inner;
    long blocks = (total + 255) / 256;
    if (blocks > 148L * 16) blocks = 148L * 16;
    ib_launch(clamped_gate_kernel, (int)blocks, 256, 0, stream, (const act_t*)gate_up, (act_t*)out, inner, total, limit,
              slope, mode);
    return ib_launch_status();
}

// ---------------------------------------------------------------------------
// Router.  logits [rows, ld] float hold n_experts router logits per row (and, with has_shared, one more column:
// the shared expert's gate).  mode 0: weights[r, e] = softmax over the `top` largest of logits[r, :] + bias among
// themselves for those experts, 0 for the others (equal logits: the lower index wins).  mode 1: the scores are
// s = sigmoid(logits + bias), the `top` largest scores are chosen (equal scores: the lower index) and
// weights[r, e] = s_e / (sum of the chosen scores + 1e-20).  mode 2: the same with the scores s = softmax(logits +
// bias) over all experts.  Either way the weights are multiplied by `scale`;
// weights[r, n_experts] = sigmoid(logits[r, n_experts]).  One warp per row.
// ---------------------------------------------------------------------------
__global__ void router_topk_kernel(const float* __restrict__ logits, long ld, const float* __restrict__ bias,
                                   int n_experts, int top, int has_shared, float* __restrict__ weights, int n_rows,
                                   int mode, float scale) {
    ib_grid_dependency_sync();
    const int lane = threadIdx.x & 31;
    const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= n_rows) return;
    const float* z = logits + (long)row * ld;
    float* w = weights + (long)row * (n_experts + has_shared);
    // a chosen expert is marked by a weight of -1 until the softmax replaces it
    for (int e = lane; e < n_experts; e += 32) w[e] = 0.0f;
    __syncwarp();
    float first = 0.0f, sum = 0.0f;
    float z_max = -INFINITY, z_den = 1.0f;      // mode 2: the softmax over all experts
    if (mode == 2) {
        for (int e = lane; e < n_experts; e += 32) z_max = fmaxf(z_max, z[e] + (bias ? bias[e] : 0.0f));
        z_max = ib_warp_max(z_max);
        float d = 0.0f;
        for (int e = lane; e < n_experts; e += 32) d += expf(z[e] + (bias ? bias[e] : 0.0f) - z_max);
        z_den = ib_warp_sum(d);
    }
    for (int k = 0; k < top; ++k) {
        float best = -INFINITY;
        int at = 0x7fffffff;
        for (int e = lane; e < n_experts; e += 32) {
            float v = z[e] + (bias ? bias[e] : 0.0f);
            if (mode == 1) v = sm_sigmoid(v);
            if (mode == 2) v = expf(v - z_max) / z_den;
            if (w[e] == 0.0f && (v > best || (v == best && e < at))) { best = v; at = e; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oa = __shfl_xor_sync(0xffffffffu, at, o);
            if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; }
        }
        if (at == 0x7fffffff) break;        // fewer experts than `top`, or nothing but NaN
        if (k == 0) first = best;
        sum += mode != 0 ? best : expf(best - first);
        if (lane == 0) w[at] = -1.0f;
        __syncwarp();
    }
    for (int e = lane; e < n_experts; e += 32)
        if (w[e] < 0.0f) {
            const float v = z[e] + (bias ? bias[e] : 0.0f);
            w[e] = (mode == 1 ? sm_sigmoid(v) / (sum + 1e-20f)
                    : mode == 2 ? expf(v - z_max) / z_den / (sum + 1e-20f) : expf(v - first) / sum) * scale;
        }
    if (has_shared && lane == 0) w[n_experts] = sm_sigmoid(z[n_experts]);
}

IB_EXPORT int ib_router_topk(const float* logits, long ld, const float* bias, int n_experts, int top, int has_shared,
                             float* weights, int n_rows, int mode, float scale, cudaStream_t stream) {
    if (n_rows <= 0) return IB_OK;
    if (n_experts <= 0 || top <= 0 || top > n_experts || logits == nullptr || weights == nullptr || mode < 0 || mode > 2 ||
        ld < n_experts + (has_shared ? 1 : 0))
        return IB_ERR_ARGUMENT;
    const int warps = 4;
    ib_launch(router_topk_kernel, (n_rows + warps - 1) / warps, 32 * warps, 0, stream, logits, ld, bias, n_experts, top,
              has_shared ? 1 : 0, weights, n_rows, mode, scale);
    return ib_launch_status();
}

// ---------------------------------------------------------------------------
// out[r, j] = silu(gate_up[r, j]) * gate_up[r, inner + j] * weights[r, e(j)]: the columns of all experts side by
// side, `ff` columns each for the n_experts routed ones (e(j) = j / ff) and the rest for the shared one
// (e(j) = n_experts).  A token's columns of experts that it did not choose become zero, so the product with the
// down matrices of all experts, side by side along its inner dimension, is the weighted sum over the chosen.
// ---------------------------------------------------------------------------
__global__ void routed_gate_kernel(const act_t* __restrict__ gate_up, const float* __restrict__ weights, int n_weights,
                                   int n_experts, int ff, act_t* __restrict__ out, int inner, long total, int act_mode,
                                   float limit, float slope) {
    ib_grid_dependency_sync();
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
        const long r = i / inner;
        const int j = (int)(i - r * inner);
        int e = j / ff;
        if (e > n_experts) e = n_experts;
        const float wt = weights[r * n_weights + e];
        float v = 0.0f;
        if (wt != 0.0f) {
            v = sm_gate_value(act_mode, ib_to_float(gate_up[r * 2 * inner + j]),
                              ib_to_float(gate_up[r * 2 * inner + inner + j]), limit, slope) * wt;
        }
        out[i] = ib_from_float<act_t>(v);
    }
}

// The same, sixteen bytes per thread and one row per blockIdx.y: for expert sizes that are multiples of that many
// elements (a thread's elements then belong to one expert).  The columns of an expert that the token did not
// choose are not read.
__global__ void routed_gate_vec_kernel(const act_t* __restrict__ gate_up, const float* __restrict__ weights,
                                       int n_weights, int n_experts, int ff, act_t* __restrict__ out, int inner,
                                       int act_mode, float limit, float slope) {
    ib_grid_dependency_sync();
    const int j = blockIdx.x * blockDim.x + threadIdx.x;
    if (j >= inner / SM_VEC) return;
    const long r = blockIdx.y;
    int e = (j * SM_VEC) / ff;
    if (e > n_experts) e = n_experts;
    const float wt = weights[r * n_weights + e];
    SmActVec o;
    if (wt != 0.0f) {
        const SmActVec g = reinterpret_cast<const SmActVec*>(gate_up + r * 2 * inner)[j];
        const SmActVec u = reinterpret_cast<const SmActVec*>(gate_up + r * 2 * inner + inner)[j];
#pragma unroll
        for (int k = 0; k < SM_VEC; ++k)
            o.v[k] = ib_from_float<act_t>(sm_gate_value(act_mode, ib_to_float(g.v[k]), ib_to_float(u.v[k]), limit,
                                                        slope) * wt);
    } else {
#pragma unroll
        for (int k = 0; k < SM_VEC; ++k) o.v[k] = ib_from_float<act_t>(0.0f);
    }
    reinterpret_cast<SmActVec*>(out + r * inner)[j] = o;
}

// clamped != 0: the experts' activation is the clamped form with `limit` and `slope` instead of silu(g) * u.
IB_EXPORT int ib_routed_gate(const void* gate_up, const float* weights, int n_weights, int n_experts, int ff, void* out,
                             int n_rows, int inner, int clamped, float limit, float slope, cudaStream_t stream) {
    if (n_rows <= 0) return IB_OK;
    if (clamped && !(limit > 0.0f)) return IB_ERR_ARGUMENT;
    const int act_mode = clamped ? 0 : 2;
    if (inner <= 0 || ff <= 0 || n_experts <= 0 || (long)n_experts * ff > inner || weights == nullptr ||
        n_weights < n_experts + ((long)n_experts * ff < inner ? 1 : 0))
        return IB_ERR_ARGUMENT;
    if (ff % SM_VEC == 0 && inner % SM_VEC == 0 && sm_aligned16(gate_up) && sm_aligned16(out)) {
        const int nv = inner / SM_VEC;
        const int threads = nv >= 256 ? 256 : ((nv + 31) / 32) * 32;
        for (int r0 = 0; r0 < n_rows; r0 += 65535) {   // blockIdx.y holds at most 65,535 rows
            const int rows = n_rows - r0 < 65535 ? n_rows - r0 : 65535;
            ib_launch(routed_gate_vec_kernel, dim3((nv + threads - 1) / threads, rows), threads, 0, stream,
                      (const act_t*)gate_up + (long)r0 * 2 * inner, weights + (long)r0 * n_weights, n_weights, n_experts,
                      ff, (act_t*)out + (long)r0 * inner, inner, act_mode, limit, slope);
        }
        return ib_launch_status();
    }
    const long total = (long)n_rows * inner;
    long blocks = (total + 255) / 256;
    if (blocks > 148L * 16) blocks = 148L * 16;
    ib_launch(routed_gate_kernel, (int)blocks, 256, 0, stream, (const act_t*)gate_up, weights, n_weights, n_experts, ff,
              (act_t*)out, inner, total, act_mode, limit, slope);
    return ib_launch_status();
}
