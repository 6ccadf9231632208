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

#define CN_VEC (16 / (int)sizeof(act_t))
struct alignas(16) CnActVec { act_t v[CN_VEC]; };
template <typename T, int N> struct alignas(sizeof(T) * N >= 16 ? 16 : sizeof(T) * N) CnVec { T v[N]; };

// N floats (a multiple of four) from or to an address that is a multiple of sixteen bytes
template <int N> __device__ __forceinline__ void cn_load(float (&dst)[N], const float* src) {
#pragma unroll
    for (int i = 0; i < N; i += 4) {
        const float4 t = *reinterpret_cast<const float4*>(src + i);
        dst[i] = t.x; dst[i + 1] = t.y; dst[i + 2] = t.z; dst[i + 3] = t.w;
    }
}
template <int N> __device__ __forceinline__ void cn_store(float* dst, const float (&src)[N]) {
#pragma unroll
    for (int i = 0; i < N; i += 4)
        *reinterpret_cast<float4*>(dst + i) = make_float4(src[i], src[i + 1], src[i + 2], src[i + 3]);
}

// ---------------------------------------------------------------------------
// out[r, c] = add_input * x[r, col + c] + sum_j w[j, c] * input(r - (taps - 1 - j), c), c < C.  w [taps, C] float
// (tap-major, so that neighbouring channels' weights are neighbours), the last tap weighs the row itself.
// shift_single (only for steps in which every request brings exactly one row): the kernel also moves the kept inputs
// on by one place, so the state is ready for the next step.  VEC: sixteen bytes per thread and access.
// ---------------------------------------------------------------------------
template <bool VEC>
__global__ void causal_conv_rows_kernel(const act_t* __restrict__ x, long ld, int col, int C, int taps,
                                        const float* __restrict__ w, float* __restrict__ state, long slot_stride,
                                        long state_off, const int* __restrict__ q_start, const int* __restrict__ slots,
                                        const int* __restrict__ row_request, act_t* __restrict__ out, long out_ld,
                                        int add_input, int shift_single) {
    ib_grid_dependency_sync();
    constexpr int V = VEC ? CN_VEC : 1;
    const int row = blockIdx.y;
    const int c0 = (blockIdx.x * blockDim.x + threadIdx.x) * V;
    if (c0 >= C) return;
    const int req = row_request[row];
    const int row0 = q_start[req];
    float* kept = taps > 1 ? state + (long)slots[req] * slot_stride + state_off : nullptr;
    float acc[V], own[V];
#pragma unroll
    for (int i = 0; i < V; ++i) acc[i] = 0.0f;
    for (int j = 0; j < taps; ++j) {
        const int t = row - (taps - 1 - j);
        float v[V], wv[V];
        if (t >= row0) {
            if constexpr (VEC) {
                const CnActVec a = *reinterpret_cast<const CnActVec*>(x + (long)t * ld + col + c0);
#pragma unroll
                for (int i = 0; i < V; ++i) v[i] = ib_to_float(a.v[i]);
            } else {
                v[0] = ib_to_float(x[(long)t * ld + col + c0]);
            }
        } else {
#pragma unroll
            for (int i = 0; i < V; ++i) v[i] = kept[(long)(taps - 1 - (row0 - t)) * C + c0 + i];
        }
        if constexpr (VEC) cn_load(wv, w + (long)j * C + c0); else wv[0] = w[(long)j * C + c0];
#pragma unroll
        for (int i = 0; i < V; ++i) acc[i] = fmaf(wv[i], v[i], acc[i]);
        if (j == taps - 1) {
#pragma unroll
            for (int i = 0; i < V; ++i) own[i] = v[i];
        }
    }
    CnActVec o;
#pragma unroll
    for (int i = 0; i < V; ++i) o.v[i] = ib_from_float<act_t>(add_input ? acc[i] + own[i] : acc[i]);
    if constexpr (VEC) *reinterpret_cast<CnActVec*>(out + (long)row * out_ld + c0) = o; else out[(long)row * out_ld + c0] = o.v[0];
    // a step in which every request brings one row: the thread that has read the channels' kept inputs moves them
    // on by one place itself, and no kernel of its own has to follow
    if (shift_single && taps > 1) {
        for (int k = 0; k + 1 < taps - 1; ++k)
#pragma unroll
            for (int i = 0; i < V; ++i) kept[(long)k * C + c0 + i] = kept[(long)(k + 1) * C + c0 + i];
#pragma unroll
        for (int i = 0; i < V; ++i) kept[(long)(taps - 2) * C + c0 + i] = own[i];
    }
}

static inline bool cn_aligned16(const void* p) { return ((uintptr_t)p & 15) == 0; }

IB_EXPORT int ib_causal_conv_rows(const void* x, long ld, int col, int C, int taps, const float* w, const float* state,
                                  long slot_stride, long state_off, const int* q_start, const int* slots,
                                  const int* row_request, void* out, long out_ld, int add_input, int shift_single,
                                  int n_rows, cudaStream_t stream) {
    if (n_rows <= 0) return IB_OK;
    if (C <= 0 || taps <= 0 || x == nullptr || w == nullptr || out == nullptr || col < 0 || ld < col + C || out_ld < C ||
        (taps > 1 && (state == nullptr || slot_stride < state_off + (long)(taps - 1) * C)))
        return IB_ERR_ARGUMENT;
    if (n_rows > 65535) return IB_ERR_UNSUPPORTED;
    const bool vec = C % CN_VEC == 0 && col % CN_VEC == 0 && ld % CN_VEC == 0 && out_ld % CN_VEC == 0 &&
                     cn_aligned16(x) && cn_aligned16(out) && cn_aligned16(w);
    const int units = vec ? C / CN_VEC : C;
    const int threads = units >= 256 ? 256 : ((units + 31) / 32) * 32;
    const dim3 grid((units + threads - 1) / threads, n_rows);
    if (vec)
        ib_launch(causal_conv_rows_kernel<true>, grid, threads, 0, stream, (const act_t*)x, ld, col, C, taps, w,
                  (float*)state, slot_stride, state_off, q_start, slots, row_request, (act_t*)out, out_ld, add_input,
                  shift_single);
    else
        ib_launch(causal_conv_rows_kernel<false>, grid, threads, 0, stream, (const act_t*)x, ld, col, C, taps, w,
                  (float*)state, slot_stride, state_off, q_start, slots, row_request, (act_t*)out, out_ld, add_input,
                  shift_single);
    return ib_launch_status();
}

// ---------------------------------------------------------------------------
// One block per row of a fused projection q | k | v (H heads of D, G heads of D, G heads of E, from column 0 on):
//   1. taps > 0: every channel goes through its causal convolution (conv_w [taps, Cq + Ck + Cv]: tap-major, so that
//      neighbouring channels' weights are neighbours; no bias);
//   2. norm_mode 1: every head of q and of k is divided by its root mean square over D and multiplied by the
//      weight [D]; norm_mode 2: all of q (all of k) is divided by one root mean square over its H * D (G * D)
//      numbers and multiplied by the weight [H * D] ([G * D]); 0: neither;
//   3. the first rot_dim numbers of every head of q and k turn by the row's position (i with i + rot_dim / 2);
//   4. q goes to q_out [rows, H, D], k and v to their pages at the row's position.  A request's last row of the step
//      clears the places behind its value in the value's page (see the kernel that stores without a convolution).
// The row lives in shared memory as floats between the steps.  VEC: sixteen bytes per thread and access (eight
// bfloat16 or four floats), for head sizes that are multiples of that many elements and aligned tensors.
// shift_single (only for steps in which every request brings exactly one row): the kernel also moves the kept inputs
// on by one place, so that no kernel of its own has to follow.
// ---------------------------------------------------------------------------
template <typename WT, bool VEC>
__global__ void conv_norm_rope_store_kernel(
    const act_t* __restrict__ proj, long ld, int H, int G, int D, int E, int taps, const float* __restrict__ conv_w,
    float* __restrict__ state, long slot_stride, long state_off, const int* __restrict__ q_start,
    const int* __restrict__ slots, const int* __restrict__ row_request, int norm_mode, const WT* __restrict__ q_weight,
    const WT* __restrict__ k_weight, float eps, const float* __restrict__ cos_table, const float* __restrict__ sin_table,
    int rot_dim, int table_rows, const int* __restrict__ positions, const int* __restrict__ block_table, int max_pages,
    int page_size, int n_pages, act_t* __restrict__ k_pages, act_t* __restrict__ v_pages, act_t* __restrict__ q_out,
    int shift_single) {
    extern __shared__ __align__(16) float cn_row[];
    __shared__ float red[64];
    ib_grid_dependency_sync();
    constexpr int V = VEC ? CN_VEC : 1;
    const int row = blockIdx.x;
    const int Cq = H * D, Ck = G * D, Cv = G * E, C = Cq + Ck + Cv;
    const int pos = positions[row];
    if (pos < 0 || (rot_dim > 0 && pos >= table_rows)) return;      // outside the tables: the row is left out
    const int req = row_request[row];
    const int row0 = q_start[req];
    float* kept = (state && taps > 1) ? state + (long)slots[req] * slot_stride + state_off : nullptr;

    // 1. the convolution (or the projection as it is)
    float ssq = 0.0f, ssk = 0.0f;
    for (int c0 = threadIdx.x * V; c0 < C; c0 += blockDim.x * V) {
        float acc[V], own[V];
#pragma unroll
        for (int i = 0; i < V; ++i) acc[i] = 0.0f;
        const int n_taps = taps > 0 ? taps : 1;
        for (int j = 0; j < n_taps; ++j) {
            const int t = row - (n_taps - 1 - j);
            float v[V];
            if (t >= row0) {
                if (VEC) {
                    const CnActVec a = *reinterpret_cast<const CnActVec*>(proj + (long)t * ld + c0);
#pragma unroll
                    for (int i = 0; i < V; ++i) v[i] = ib_to_float(a.v[i]);
                } else {
                    v[0] = ib_to_float(proj[(long)t * ld + c0]);
                }
            } else {
#pragma unroll
                for (int i = 0; i < V; ++i) v[i] = kept[(long)(n_taps - 1 - (row0 - t)) * C + c0 + i];
            }
            if (j == n_taps - 1) {
#pragma unroll
                for (int i = 0; i < V; ++i) own[i] = v[i];
            }
            if (taps > 0) {
                float wv[V];
                if constexpr (VEC) cn_load(wv, conv_w + (long)j * C + c0); else wv[0] = conv_w[(long)j * C + c0];
#pragma unroll
                for (int i = 0; i < V; ++i) acc[i] = fmaf(wv[i], v[i], acc[i]);
            } else {
#pragma unroll
                for (int i = 0; i < V; ++i) acc[i] = v[i];
            }
        }
        if constexpr (VEC) cn_store(cn_row + c0, acc); else cn_row[c0] = acc[0];
#pragma unroll
        for (int i = 0; i < V; ++i) {
            if (c0 + i < Cq) ssq += acc[i] * acc[i];
            else if (c0 + i < Cq + Ck) ssk += acc[i] * acc[i];
        }
        if (shift_single && kept != nullptr) {        // this thread alone has read these channels' kept inputs
            for (int k = 0; k + 1 < taps - 1; ++k)
#pragma unroll
                for (int i = 0; i < V; ++i) kept[(long)k * C + c0 + i] = kept[(long)(k + 1) * C + c0 + i];
#pragma unroll
            for (int i = 0; i < V; ++i) kept[(long)(taps - 2) * C + c0 + i] = own[i];
        }
    }
    // 2. the norms
    if (norm_mode == 2) {
        {   // the two sums of squares over the block at once: one meeting instead of two
            const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = (blockDim.x + 31) >> 5;
            ssq = ib_warp_sum(ssq);
            ssk = ib_warp_sum(ssk);
            if (lane == 0) { red[warp] = ssq; red[32 + warp] = ssk; }
            __syncthreads();
            ssq = ib_warp_sum(lane < n_warps ? red[lane] : 0.0f);
            ssk = ib_warp_sum(lane < n_warps ? red[32 + lane] : 0.0f);
        }
        const float inv_q = 1.0f / sqrtf(ssq / (float)Cq + eps), inv_k = 1.0f / sqrtf(ssk / (float)Ck + eps);
        for (int c0 = threadIdx.x * V; c0 < Cq + Ck; c0 += blockDim.x * V) {    // the thread that wrote the places reads them
            const bool is_q = c0 < Cq;       // a thread's V numbers lie in one head, so in one projection
            const float inv = is_q ? inv_q : inv_k;
            const WT* wp = is_q ? q_weight + c0 : k_weight + (c0 - Cq);
            if constexpr (VEC) {
                const CnVec<WT, V> wv = *reinterpret_cast<const CnVec<WT, V>*>(wp);
                float r[V];
                cn_load(r, cn_row + c0);
#pragma unroll
                for (int i = 0; i < V; ++i) r[i] *= inv * ib_to_float(wv.v[i]);
                cn_store(cn_row + c0, r);
            } else {
                cn_row[c0] *= inv * ib_to_float(wp[0]);
            }
        }
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
    for (int c0 = threadIdx.x * V; c0 < Cq + Ck; c0 += blockDim.x * V) {
        const int head = c0 / D, j0 = c0 - head * D;      // a thread's V numbers lie in one head
        CnActVec o;
        if constexpr (VEC) {      // half is a multiple of V: the V numbers turn with V partners half a rotation away
            float r[V];
            cn_load(r, cn_row + c0);
            if (j0 < rot_dim) {
                const bool lower = j0 < half;
                const int tj = lower ? j0 : j0 - half;
                float partner[V], cv[V], sv[V];
                cn_load(partner, cn_row + (lower ? c0 + half : c0 - half));
                cn_load(cv, cs + tj);
                cn_load(sv, sn + tj);
#pragma unroll
                for (int i = 0; i < V; ++i) r[i] = lower ? r[i] * cv[i] - partner[i] * sv[i] : partner[i] * sv[i] + r[i] * cv[i];
            }
#pragma unroll
            for (int i = 0; i < V; ++i) o.v[i] = ib_from_float<act_t>(r[i]);
        } else {
            const int c = c0, j = j0;
            float r = cn_row[c];
            if (j < half) r = r * cs[j] - cn_row[c + half] * sn[j];
            else if (j < rot_dim) r = cn_row[c - half] * sn[j - half] + r * cs[j - half];
            o.v[0] = ib_from_float<act_t>(r);
        }
        act_t* dst = head < H ? q_out + ((long)row * H + head) * D + j0
                              : (kv_place >= 0 ? k_pages + (kv_place + (long)(head - H) * page_size) * D + j0 : nullptr);
        if (dst == nullptr) continue;
        if (VEC) *reinterpret_cast<CnActVec*>(dst) = o; else dst[0] = o.v[0];
    }
    if (kv_place < 0) return;
    for (int c0 = threadIdx.x * V; c0 < Cv; c0 += blockDim.x * V) {
        const int g = c0 / E, j0 = c0 - g * E;
        CnActVec o;
        if constexpr (VEC) {
            float r[V];
            cn_load(r, cn_row + Cq + Ck + c0);
#pragma unroll
            for (int i = 0; i < V; ++i) o.v[i] = ib_from_float<act_t>(r[i]);
        } else {
            o.v[0] = ib_from_float<act_t>(cn_row[Cq + Ck + c0]);
        }
        act_t* dst = v_pages + (kv_place + (long)g * page_size) * E + j0;
        if (VEC) *reinterpret_cast<CnActVec*>(dst) = o; else dst[0] = o.v[0];
    }
    const bool last = row + 1 >= (int)gridDim.x || row_request[row + 1] != req;
    const int behind = last ? (page_size - 1 - pos % page_size) * E : 0;
    for (int g = 0; g < G && behind > 0; ++g) {
        act_t* dst = v_pages + (kv_place + (long)g * page_size) * E + E;
        for (int j = threadIdx.x; j < behind; j += blockDim.x) dst[j] = ib_from_float<act_t>(0.0f);
    }
}

IB_EXPORT int ib_conv_norm_rope_store(const void* proj, long ld, int n_rows, int H, int G, int D, int E, int taps,
                                      const float* conv_w, float* state, long slot_stride, long state_off,
                                      const int* q_start, const int* slots, const int* row_request, int norm_mode,
                                      const void* q_weight, const void* k_weight, int weight_is_f32, float eps,
                                      const float* cos_table, const float* sin_table, int rot_dim, int table_rows,
                                      const int* positions, const int* block_table, int max_pages, int page_size,
                                      int n_pages, void* k_pages, void* v_pages, void* q_out, int shift_single,
                                      cudaStream_t stream) {
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
    static IbDeviceSet sets[4];
    const bool vec = D % CN_VEC == 0 && E % CN_VEC == 0 && ld % CN_VEC == 0 && cn_aligned16(proj) &&
                     cn_aligned16(q_out) && cn_aligned16(k_pages) && cn_aligned16(v_pages) &&
                     (rot_dim / 2) % CN_VEC == 0 && cn_aligned16(conv_w) && cn_aligned16(cos_table) &&
                     cn_aligned16(sin_table) && cn_aligned16(q_weight) && cn_aligned16(k_weight);
    const long units = vec ? C / CN_VEC : C;
    const int threads = units >= 512 ? 512 : (units >= 256 ? 256 : (units > 64 ? 128 : 64));
#define IB_CNRS(WT, VEC, SET)                                                                                         \
    do {                                                                                                              \
        if (smem > 48 * 1024) {                                                                                       \
            const int e = ib_allow_dynamic_smem(sets[SET], conv_norm_rope_store_kernel<WT, VEC>, 200 * 1024);         \
            if (e != IB_OK) return e;                                                                                 \
        }                                                                                                             \
        ib_launch(conv_norm_rope_store_kernel<WT, VEC>, n_rows, threads, smem, stream, (const act_t*)proj, ld, H, G,  \
                  D, E, taps, conv_w, state, slot_stride, state_off, q_start, slots, row_request, norm_mode,          \
                  (const WT*)q_weight, (const WT*)k_weight, eps, cos_table, sin_table, rot_dim, table_rows, positions, \
                  block_table, max_pages, page_size, n_pages, (act_t*)k_pages, (act_t*)v_pages, (act_t*)q_out,        \
                  shift_single);                                                                                      \
    } while (0)
    if (weight_is_f32) {
        if (vec) IB_CNRS(float, true, 0); else IB_CNRS(float, false, 1);
    } else {
        if (vec) IB_CNRS(__nv_bfloat16, true, 2); else IB_CNRS(__nv_bfloat16, false, 3);
    }
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
