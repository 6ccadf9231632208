// Short causal convolutions over a request's rows, and what attention layers that have them need around them.
// Every sum and norm is float in both builds; act_t is what the projections hand in and what the next product reads.
//
//   convolution on rows       out[r, c] = (x[r, c]) + sum_j w[c, j] * input(r - (taps - 1 - j), c): the sub-layer input
//                             that is replaced by itself plus its convolution, or the convolution alone
//   convolution, norm,        one pass over a fused q | k | v projection: the convolution per channel, the root mean
//   rotation and store        square over a whole projection (all heads at once) or per head, the rotation by
//                             position, q to a dense tensor, k and v into their pages
//   blend of columns          x[r, col + c] <- (1 - lambda) x[r, col + c] + lambda other[r, c]: values mixed with an
//                             earlier layer's values of the same token
//
// input(t, c) is this step's row t if t is a row of the same request, and else what the request's state keeps: its
// last taps - 1 inputs, oldest first, [taps - 1, C] floats at state_off of its slot (zeros for a new request).
#include "common.cuh"

// ---------------------------------------------------------------------------
// out[r, c] = add_input * x[r, col + c] + sum_j w[c, j] * input(r - (taps - 1 - j), c), c < C.  w [C, taps] float, the
// last tap weighs the row itself.
// ---------------------------------------------------------------------------
__global__ void causal_conv_rows_kernel(const act_t* __restrict__ x, long ld, int col, int C, int taps,
                                        const float* __restrict__ w, const float* __restrict__ state, long slot_stride,
                                        long state_off, const int* __restrict__ q_start, const int* __restrict__ slots,
                                        const int* __restrict__ row_request, act_t* __restrict__ out, long out_ld,
                                        int add_input) {
    ib_grid_dependency_sync();
    const int row = blockIdx.y;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= C) return;
    const int req = row_request[row];
    const int row0 = q_start[req];
    const float* kept = state + (long)slots[req] * slot_stride + state_off;
    float acc = add_input ? ib_to_float(x[(long)row * ld + col + c]) : 0.0f;
    for (int j = 0; j < taps; ++j) {
        const int t = row - (taps - 1 - j);
        float v;
        if (t >= row0) v = ib_to_float(x[(long)t * ld + col + c]);
        else v = kept[(long)(taps - 1 - (row0 - t)) * C + c];
        acc = fmaf(w[(long)c * taps + j], v, acc);
    }
    out[(long)row * out_ld + c] = ib_from_float<act_t>(acc);
}

IB_EXPORT int ib_causal_conv_rows(const void* x, long ld, int col, int C, int taps, const float* w, const float* state,
                                  long slot_stride, long state_off, const int* q_start, const int* slots,
                                  const int* row_request, void* out, long out_ld, int add_input, int n_rows,
                                  cudaStream_t stream) {
    if (n_rows <= 0) return IB_OK;
    if (C <= 0 || taps <= 0 || x == nullptr || w == nullptr || out == nullptr || col < 0 || ld < col + C || out_ld < C ||
        (taps > 1 && (state == nullptr || slot_stride < state_off + (long)(taps - 1) * C)))
        return IB_ERR_ARGUMENT;
    if (n_rows > 65535) return IB_ERR_UNSUPPORTED;
    const int threads = C >= 256 ? 256 : ((C + 31) / 32) * 32;
    ib_launch(causal_conv_rows_kernel, dim3((C + threads - 1) / threads, n_rows), threads, 0, stream, (const act_t*)x,
              ld, col, C, taps, w, state, slot_stride, state_off, q_start, slots, row_request, (act_t*)out, out_ld,
              add_input);
    return ib_launch_status();
}

// ---------------------------------------------------------------------------
// One block per row of a fused projection q | k | v (H heads of D, G heads of D, G heads of E, from column 0 on):
//   1. taps > 0: every channel goes through its causal convolution (conv_w [Cq + Ck + Cv, taps], no bias);
//   2. norm_mode 1: every head of q and of k is divided by its root mean square over D and multiplied by the
//      weight [D]; norm_mode 2: all of q (all of k) is divided by one root mean square over its H * D (G * D)
//      numbers and multiplied by the weight [H * D] ([G * D]); 0: neither;
//   3. the first rot_dim numbers of every head of q and k turn by the row's position (i with i + rot_dim / 2);
//   4. q goes to q_out [rows, H, D], k and v to their pages at the row's position.  A request's last row of the step
//      clears the places behind its value in the value's page (see the kernel that stores without a convolution).
// The row lives in shared memory as floats between the steps.
// ---------------------------------------------------------------------------
template <typename WT>
__global__ void conv_norm_rope_store_kernel(
    const act_t* __restrict__ proj, long ld, int H, int G, int D, int E, int taps, const float* __restrict__ conv_w,
    const float* __restrict__ state, long slot_stride, long state_off, const int* __restrict__ q_start,
    const int* __restrict__ slots, const int* __restrict__ row_request, int norm_mode, const WT* __restrict__ q_weight,
    const WT* __restrict__ k_weight, float eps, const float* __restrict__ cos_table, const float* __restrict__ sin_table,
    int rot_dim, int table_rows, const int* __restrict__ positions, const int* __restrict__ block_table, int max_pages,
    int page_size, int n_pages, act_t* __restrict__ k_pages, act_t* __restrict__ v_pages, act_t* __restrict__ q_out) {
    extern __shared__ float cn_row[];
    __shared__ float red[32];
    ib_grid_dependency_sync();
    const int row = blockIdx.x;
    const int Cq = H * D, Ck = G * D, Cv = G * E, C = Cq + Ck + Cv;
    const int pos = positions[row];
    if (pos < 0 || (rot_dim > 0 && pos >= table_rows)) return;      // outside the tables: the row is left out
    const int req = row_request[row];
    const int row0 = q_start[req];
    const float* kept = state ? state + (long)slots[req] * slot_stride + state_off : nullptr;

    // 1. the convolution (or the projection as it is)
    float ssq = 0.0f, ssk = 0.0f;
    for (int c = threadIdx.x; c < C; c += blockDim.x) {
        float acc;
        if (taps > 0) {
            acc = 0.0f;
            for (int j = 0; j < taps; ++j) {
                const int t = row - (taps - 1 - j);
                float v;
                if (t >= row0) v = ib_to_float(proj[(long)t * ld + c]);
                else v = kept[(long)(taps - 1 - (row0 - t)) * C + c];
                acc = fmaf(conv_w[(long)c * taps + j], v, acc);
            }
        } else {
            acc = ib_to_float(proj[(long)row * ld + c]);
        }
        cn_row[c] = acc;
        if (c < Cq) ssq += acc * acc;
        else if (c < Cq + Ck) ssk += acc * acc;
    }
    // 2. the norms
    if (norm_mode == 2) {
        ssq = ib_block_sum(ssq, red);
        ssk = ib_block_sum(ssk, red);
        const float inv_q = 1.0f / sqrtf(ssq / (float)Cq + eps), inv_k = 1.0f / sqrtf(ssk / (float)Ck + eps);
        for (int c = threadIdx.x; c < Cq + Ck; c += blockDim.x)      // the thread that wrote the place reads it
            cn_row[c] *= c < Cq ? inv_q * ib_to_float(q_weight[c]) : inv_k * ib_to_float(k_weight[c - Cq]);
        __syncthreads();
    } else if (norm_mode == 1) {
        __syncthreads();
        const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
        for (int head = warp; head < H + G; head += n_warps) {
            float* hv = cn_row + (long)head * D;
            const WT* w = head < H ? q_weight : k_weight;
            float ss = 0.0f;
            for (int j = lane; j < D; j += 32) ss += hv[j] * hv[j];
            ss = ib_warp_sum(ss);
            const float inv = 1.0f / sqrtf(ss / (float)D + eps);
            for (int j = lane; j < D; j += 32) hv[j] *= inv * (w ? ib_to_float(w[j]) : 1.0f);
        }
        __syncthreads();
    } else {
        __syncthreads();
    }
    // 3., 4. rotation and store
    long kv_place = -1;      // (page, key/value head 0, place in the page) counted in heads' rows
    {
        const int page = pos / page_size < max_pages ? block_table[(long)req * max_pages + pos / page_size] : -1;
        if (page >= 0 && page < n_pages) kv_place = (long)page * G * page_size + (pos % page_size);
    }
    const int half = rot_dim / 2;
    const float* cs = rot_dim > 0 ? cos_table + (long)pos * half : nullptr;
    const float* sn = rot_dim > 0 ? sin_table + (long)pos * half : nullptr;
    for (int c = threadIdx.x; c < Cq + Ck; c += blockDim.x) {
        const int head = c / D, j = c - head * D;
        float o = cn_row[c];
        if (j < half) o = o * cs[j] - cn_row[c + half] * sn[j];
        else if (j < rot_dim) o = cn_row[c - half] * sn[j - half] + o * cs[j - half];
        if (head < H) q_out[((long)row * H + head) * D + j] = ib_from_float<act_t>(o);
        else if (kv_place >= 0) k_pages[(kv_place + (long)(head - H) * page_size) * D + j] = ib_from_float<act_t>(o);
    }
    if (kv_place < 0) return;
    const bool last = row + 1 >= (int)gridDim.x || row_request[row + 1] != req;
    const int behind = last ? (page_size - 1 - pos % page_size) * E : 0;
    for (int c = threadIdx.x; c < Cv; c += blockDim.x) {
        const int g = c / E, j = c - g * E;
        v_pages[(kv_place + (long)g * page_size) * E + j] = ib_from_float<act_t>(cn_row[Cq + Ck + c]);
    }
    for (int g = 0; g < G; ++g) {
        act_t* dst = v_pages + (kv_place + (long)g * page_size) * E + E;
        for (int j = threadIdx.x; j < behind; j += blockDim.x) dst[j] = ib_from_float<act_t>(0.0f);
    }
}

IB_EXPORT int ib_conv_norm_rope_store(const void* proj, long ld, int n_rows, int H, int G, int D, int E, int taps,
                                      const float* conv_w, const float* state, long slot_stride, long state_off,
                                      const int* q_start, const int* slots, const int* row_request, int norm_mode,
                                      const void* q_weight, const void* k_weight, int weight_is_f32, float eps,
                                      const float* cos_table, const float* sin_table, int rot_dim, int table_rows,
                                      const int* positions, const int* block_table, int max_pages, int page_size,
                                      int n_pages, void* k_pages, void* v_pages, void* q_out, cudaStream_t stream) {
    if (n_rows <= 0) return IB_OK;
    if (H <= 0 || G <= 0 || D <= 0 || E <= 0 || taps < 0 || rot_dim < 0 || rot_dim > D || (rot_dim & 1) ||
        norm_mode < 0 || norm_mode > 2 || page_size <= 0 || max_pages <= 0 || proj == nullptr || q_out == nullptr ||
        k_pages == nullptr || v_pages == nullptr)
        return IB_ERR_ARGUMENT;
    const long C = (long)H * D + (long)G * (D + E);
    if (ld < C) return IB_ERR_ARGUMENT;
    if (taps > 0 && conv_w == nullptr) return IB_ERR_ARGUMENT;
    if (taps > 1 && (state == nullptr || slot_stride < state_off + (long)(taps - 1) * C)) return IB_ERR_ARGUMENT;
    if (norm_mode == 2 && (q_weight == nullptr || k_weight == nullptr)) return IB_ERR_ARGUMENT;
    if (rot_dim > 0 && (cos_table == nullptr || sin_table == nullptr || table_rows <= 0)) return IB_ERR_ARGUMENT;
    const size_t smem = (size_t)C * sizeof(float);
    if (smem > 200 * 1024) return IB_ERR_UNSUPPORTED;
    static IbDeviceSet set_f, set_b;
    const int threads = C >= 2048 ? 512 : 256;
#define IB_CNRS(WT, SET)                                                                                              \
    do {                                                                                                              \
        if (smem > 48 * 1024) {                                                                                       \
            const int e = ib_allow_dynamic_smem(SET, conv_norm_rope_store_kernel<WT>, 200 * 1024);                    \
            if (e != IB_OK) return e;                                                                                 \
        }                                                                                                             \
        ib_launch(conv_norm_rope_store_kernel<WT>, n_rows, threads, smem, stream, (const act_t*)proj, ld, H, G, D, E, \
                  taps, conv_w, state, slot_stride, state_off, q_start, slots, row_request, norm_mode,                \
                  (const WT*)q_weight, (const WT*)k_weight, eps, cos_table, sin_table, rot_dim, table_rows, positions, \
                  block_table, max_pages, page_size, n_pages, (act_t*)k_pages, (act_t*)v_pages, (act_t*)q_out);       \
    } while (0)
    if (weight_is_f32) IB_CNRS(float, set_f); else IB_CNRS(__nv_bfloat16, set_b);
#undef IB_CNRS
    return ib_launch_status();
}

// ---------------------------------------------------------------------------
// x[r, col + c] <- (1 - lambda) x[r, col + c] + lambda other[r, c] for c < C, in place; lambda is one float on the
// device (a learned number), other has the row stride other_ld.
// ---------------------------------------------------------------------------
__global__ void blend_columns_kernel(act_t* __restrict__ x, long ld, int col, int C, const act_t* __restrict__ other,
                                     long other_ld, const float* __restrict__ lambda, long total) {
    ib_grid_dependency_sync();
    const float lam = *lambda;
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
        const long r = i / C;
        const int c = (int)(i - r * C);
        act_t* p = x + r * ld + col + c;
        *p = ib_from_float<act_t>((1.0f - lam) * ib_to_float(*p) + lam * ib_to_float(other[r * other_ld + c]));
    }
}

IB_EXPORT int ib_blend_columns(void* x, long ld, int col, int C, const void* other, long other_ld, const float* lambda,
                               int n_rows, cudaStream_t stream) {
    if (n_rows <= 0) return IB_OK;
    if (C <= 0 || col < 0 || ld < col + C || other_ld < C || x == nullptr || other == nullptr || lambda == nullptr)
        return IB_ERR_ARGUMENT;
    const long total = (long)n_rows * C;
    long blocks = (total + 255) / 256;
    if (blocks > 148L * 16) blocks = 148L * 16;
    ib_launch(blend_columns_kernel, (int)blocks, 256, 0, stream, (act_t*)x, ld, col, C, (const act_t*)other, other_ld,
              lambda, total);
    return ib_launch_status();
}
