// A matrix state per head that fades and is then corrected towards the value at the key (the gated delta rule),
// carried from token to token:
//
//     S  <- fade_t S                          S is [D, E] per head
//     u   = beta_t (v_t - S^T k_t)            what the state does not yet answer for this key
//     S  <- S + k_t u^T
//     o_t = S^T q_t                           the read-out sees the token's own write
//
// fade and beta are one number per (token, head).  q and k may be shared by the heads of a group (head h reads group
// h / (H / G)) and may be made unit vectors here: x / sqrt(sum(x^2) + unit_eps), q then times q_scale.
//
// Everything is float in both builds: the kernels before this one hand in q, k and v as float rows, and the state
// lives in float.  A request's rows are walked in order, one token after the other, so a result does not depend
// on how the prompt was cut into steps or on what else the step holds.
//
// Work split: S^T k needs a whole column of S for every token, so a column is not cut over warps: a warp owns 8
// columns, and the 4 lanes that share a column own RL consecutive rows each (RL = 8, 16, 32 or 64 by D), in
// registers.  A block holds 2 or 4 such warps of one (request, head).  What a token costs is the chain from one
// state to the next, so the chain is kept short: the read-out is taken from the state before the write,
//     o_t = S_t^T q_t = fade_t (S_(t-1)^T q_t) + (k_t . q_t) u_t,
// so that S_(t-1)^T k_t and S_(t-1)^T q_t are one pass over the registers with eight sums in flight and one pair of
// shuffles for both; k_t . q_t and the factors that make q and k unit vectors are one number each per token, made
// once per chunk, and multiply the sums instead of the vectors; the next token's q and k are fetched into registers
// while this token's sums are made.  Tokens go in chunks of 16 through shared memory, two buffers: the next chunk's
// q, k, v, fade and beta are on their way (cp.async) while the chunk before is walked.  In shared memory a lane's RL
// rows of q and k are followed by four unused floats, so that the four lanes of a column read different banks.  A
// step of single tokens takes chunks of one.
//
// State of one slot: S as [H, D, E] floats (E contiguous) from the slot's first float on.
#include "common.cuh"

#define GD_COLS 8      // columns of S per warp
#define GD_PARTS 4     // lanes that share a column
#define GD_PAD 4       // floats between two lanes' rows of q and k in shared memory

__device__ __forceinline__ void gd_copy4(float* dst, const float* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((unsigned)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void gd_copy16(float* dst, const float* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((unsigned)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}

// VEC: 4 where q, k and v rows can be fetched sixteen bytes at a time (the host checks sizes and alignment), else 1.
template <int CH, int RL, int VEC>
__global__ void delta_scan_kernel(const float* __restrict__ x, long ld, int q_col, int k_col, int v_col, int G,
                                  const float* __restrict__ fade, long fade_ld, const float* __restrict__ beta,
                                  long beta_ld, float unit_eps, float q_scale, float* __restrict__ state,
                                  long slot_stride, const int* __restrict__ q_start, const int* __restrict__ slots,
                                  float* __restrict__ out, int H, int D, int E) {
    extern __shared__ __align__(16) float smem[];
    ib_grid_dependency_sync();
    constexpr int Dp = (RL + GD_PAD) * GD_PARTS;                  // a token's q or k in shared memory
    constexpr bool AHEAD = RL <= 32 && CH > 1;                    // with 64 rows per lane a second pair does not fit
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
    const int col = lane & (GD_COLS - 1), part = lane / GD_COLS;
    const int cols = n_warps * GD_COLS;                           // columns of the block
    const int h = blockIdx.y, r = blockIdx.z, e0 = blockIdx.x * cols, ec = warp * GD_COLS + col;
    const int g = h / (H / G);
    const int row0 = q_start[r], row1 = q_start[r + 1];
    if (row1 <= row0) return;                                     // the whole block leaves
    // q [CH][Dp], k [CH][Dp], v [CH][cols], fade [CH], beta [CH]; the second buffer starts on a 16-byte boundary too
    const int buf_floats = (2 * CH * Dp + CH * cols + 2 * CH + 3) & ~3;
    float* o_s = smem + 2 * buf_floats;                           // [CH][cols]
    float* qn_s = o_s + CH * cols;                                // [CH] what q's sums are multiplied by
    float* kn_s = qn_s + CH;                                      // [CH] what k's sums are multiplied by
    float* kq_s = kn_s + CH;                                      // [CH] k . q as they were fetched
    // what no copy writes stays zero: the rows beyond D, the floats between the lanes' rows, the columns beyond E
    for (int i = threadIdx.x; i < 2 * buf_floats; i += blockDim.x) smem[i] = 0.0f;
    __syncthreads();
    auto place = [](int d) { return (d / RL) * (RL + GD_PAD) + (d % RL); };      // where row d of q or k lies

    float* st = state + (long)slots[r] * slot_stride + (long)h * D * E;
    const bool col_ok = e0 + ec < E;
    const int dl = part * RL, dl_s = part * (RL + GD_PAD);
    float S[RL];
#pragma unroll
    for (int i = 0; i < RL; ++i) S[i] = (col_ok && dl + i < D) ? st[(long)(dl + i) * E + e0 + ec] : 0.0f;
    const int e_n = min(cols, E - e0);                            // this block's columns that exist

    auto fetch = [&](int c0, int buf) {
        const int nc = min(CH, row1 - c0);
        float* q_s = smem + buf * buf_floats;
        float* k_s = q_s + CH * Dp;
        float* v_s = k_s + CH * Dp;
        float* g_s = v_s + CH * cols;
        if (VEC == 4) {
            const int d4 = D >> 2;
            for (int idx = threadIdx.x; idx < nc * d4; idx += blockDim.x) {
                const int t = idx / d4, d = (idx - t * d4) << 2;
                const float* xr = x + (long)(c0 + t) * ld + g * D + d;
                gd_copy16(q_s + t * Dp + place(d), xr + q_col);
                gd_copy16(k_s + t * Dp + place(d), xr + k_col);
            }
            const int e4 = e_n >> 2;
            for (int idx = threadIdx.x; idx < nc * e4; idx += blockDim.x) {
                const int t = idx / e4, e = (idx - t * e4) << 2;
                gd_copy16(v_s + t * cols + e, x + (long)(c0 + t) * ld + v_col + h * E + e0 + e);
            }
        } else {
            for (int idx = threadIdx.x; idx < nc * D; idx += blockDim.x) {
                const int t = idx / D, d = idx - t * D;
                const float* xr = x + (long)(c0 + t) * ld + g * D + d;
                gd_copy4(q_s + t * Dp + place(d), xr + q_col);
                gd_copy4(k_s + t * Dp + place(d), xr + k_col);
            }
            for (int idx = threadIdx.x; idx < nc * e_n; idx += blockDim.x) {
                const int t = idx / e_n, e = idx - t * e_n;
                gd_copy4(v_s + t * cols + e, x + (long)(c0 + t) * ld + v_col + h * E + e0 + e);
            }
        }
        if (threadIdx.x < nc) {
            gd_copy4(g_s + threadIdx.x, fade + (long)(c0 + threadIdx.x) * fade_ld + h);
            gd_copy4(g_s + CH + threadIdx.x, beta + (long)(c0 + threadIdx.x) * beta_ld + h);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    fetch(row0, 0);

    int buf = 0;
    for (int c0 = row0; c0 < row1; c0 += CH, buf ^= 1) {
        const int nc = min(CH, row1 - c0);
        if (c0 + CH < row1) {
            fetch(c0 + CH, buf ^ 1);
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();
        const float* q_s = smem + buf * buf_floats;
        const float* k_s = q_s + CH * Dp;
        const float* v_s = k_s + CH * Dp;
        const float* g_s = v_s + CH * cols;
        // ---- three numbers per token: the unit factors of q and k, and k . q (a warp per token) ---------------
        for (int t = warp; t < nc; t += n_warps) {
            float sq = 0.0f, sk = 0.0f, kq = 0.0f;
            for (int d = lane; d < D; d += 32) {
                const float a = q_s[t * Dp + place(d)], b = k_s[t * Dp + place(d)];
                sq = fmaf(a, a, sq);
                sk = fmaf(b, b, sk);
                kq = fmaf(a, b, kq);
            }
            sq = ib_warp_sum(sq);
            sk = ib_warp_sum(sk);
            kq = ib_warp_sum(kq);
            if (lane == 0) {
                qn_s[t] = unit_eps >= 0.0f ? q_scale / sqrtf(sq + unit_eps) : q_scale;
                kn_s[t] = unit_eps >= 0.0f ? 1.0f / sqrtf(sk + unit_eps) : 1.0f;
                kq_s[t] = kq;
            }
        }
        __syncthreads();
        // ---- the tokens, one after the other ------------------------------------------------------------------
        auto load = [&](float (&kd)[RL], float (&qd)[RL], int t) {
            const float4* k4 = reinterpret_cast<const float4*>(k_s + t * Dp + dl_s);
            const float4* q4 = reinterpret_cast<const float4*>(q_s + t * Dp + dl_s);
#pragma unroll
            for (int i = 0; i < RL / 4; ++i) {
                const float4 k = k4[i], q = q4[i];
                kd[4 * i + 0] = k.x; kd[4 * i + 1] = k.y; kd[4 * i + 2] = k.z; kd[4 * i + 3] = k.w;
                qd[4 * i + 0] = q.x; qd[4 * i + 1] = q.y; qd[4 * i + 2] = q.z; qd[4 * i + 3] = q.w;
            }
        };
        // one token with its q and k in registers; the next token's are fetched into the other pair meanwhile
        auto step = [&](const float (&kc)[RL], const float (&qc)[RL], float (&kx)[RL], float (&qx)[RL], int t) {
            if (AHEAD && t + 1 < nc) load(kx, qx, t + 1);
            const float fd = g_s[t], bt = g_s[CH + t], qn = qn_s[t], kn = kn_s[t], kq = kq_s[t];
            const float vt = v_s[t * cols + ec];
            float d0 = 0.0f, d1 = 0.0f, d2 = 0.0f, d3 = 0.0f, a0 = 0.0f, a1 = 0.0f, a2 = 0.0f, a3 = 0.0f;
#pragma unroll
            for (int i = 0; i < RL / 4; ++i) {
                d0 = fmaf(S[4 * i + 0], kc[4 * i + 0], d0); a0 = fmaf(S[4 * i + 0], qc[4 * i + 0], a0);
                d1 = fmaf(S[4 * i + 1], kc[4 * i + 1], d1); a1 = fmaf(S[4 * i + 1], qc[4 * i + 1], a1);
                d2 = fmaf(S[4 * i + 2], kc[4 * i + 2], d2); a2 = fmaf(S[4 * i + 2], qc[4 * i + 2], a2);
                d3 = fmaf(S[4 * i + 3], kc[4 * i + 3], d3); a3 = fmaf(S[4 * i + 3], qc[4 * i + 3], a3);
            }
            float dot = (d0 + d1) + (d2 + d3), red = (a0 + a1) + (a2 + a3);
            dot += __shfl_xor_sync(0xffffffffu, dot, GD_COLS);
            red += __shfl_xor_sync(0xffffffffu, red, GD_COLS);
            dot += __shfl_xor_sync(0xffffffffu, dot, 2 * GD_COLS);
            red += __shfl_xor_sync(0xffffffffu, red, 2 * GD_COLS);
            // S^T k of the faded state is fade times that of the state before; k's unit factor multiplies the sum
            const float u = bt * (vt - fd * dot * kn);
            const float uk = u * kn;
#pragma unroll
            for (int i = 0; i < RL; ++i) S[i] = fmaf(kc[i], uk, fd * S[i]);
            // the read-out of the state after the write, from the sums over the state before it
            if (part == 0) o_s[t * cols + ec] = qn * fmaf(uk, kq, fd * red);
        };
        if constexpr (AHEAD) {
            float ka[RL], qa[RL], kb[RL], qb[RL];
            load(ka, qa, 0);
            for (int t = 0; t < nc; t += 2) {
                step(ka, qa, kb, qb, t);
                if (t + 1 < nc) step(kb, qb, ka, qa, t + 1);
            }
        } else {
            float ka[RL], qa[RL];
            for (int t = 0; t < nc; ++t) {
                load(ka, qa, t);
                step(ka, qa, ka, qa, t);
            }
        }
        __syncthreads();
        for (int idx = threadIdx.x; idx < nc * cols; idx += blockDim.x) {
            const int t = idx / cols, e = idx - t * cols;
            if (e0 + e < E) out[((long)(c0 + t) * H + h) * E + e0 + e] = o_s[idx];
        }
        __syncthreads();       // before the next turn's copies overwrite this buffer
    }
#pragma unroll
    for (int i = 0; i < RL; ++i)
        if (col_ok && dl + i < D) st[(long)(dl + i) * E + e0 + ec] = S[i];
}

static IbDeviceSet delta_scan_smem_set[2];      // only the form of 16 tokens and 64 rows per lane needs more than 48 KB

// x [rows, ld] float holds q and k as [G, D] and v as [H, E] from columns q_col, k_col, v_col on.  fade and beta
// [rows, *_ld] float, one number per head.  unit_eps >= 0: q and k are divided by sqrt(sum of squares + unit_eps)
// per head; q is multiplied by q_scale either way.  out [rows, H, E] float.  max_rows: the most rows that a request
// brings (1: the form for steps of single tokens).
IB_EXPORT int ib_delta_scan(const float* x, long ld, int q_col, int k_col, int v_col, int G, const float* fade,
                            long fade_ld, const float* beta, long beta_ld, float unit_eps, float q_scale, float* state,
                            long slot_stride, const int* q_start, const int* slots, int n_requests, float* out, int H,
                            int D, int E, int max_rows, cudaStream_t stream) {
    if (n_requests <= 0) return IB_OK;
    if (H <= 0 || D <= 0 || E <= 0 || G <= 0 || H % G || x == nullptr || fade == nullptr || beta == nullptr ||
        state == nullptr || out == nullptr || slot_stride < (long)H * D * E)
        return IB_ERR_ARGUMENT;
    if (D > 64 * GD_PARTS || H > 65535 || n_requests > 65535) return IB_ERR_UNSUPPORTED;
    const int ch = max_rows == 1 ? 1 : 16;
    const int rl = D <= 8 * GD_PARTS ? 8 : (D <= 16 * GD_PARTS ? 16 : (D <= 32 * GD_PARTS ? 32 : 64));
    // two warps (16 columns) per block where four would leave most SMs without a block
    int n_warps = (E + GD_COLS - 1) / GD_COLS;
    if (n_warps > 4) n_warps = 4;
    if (n_warps == 4 && ch > 1 && (long)((E + 31) / 32) * H * n_requests < 120) n_warps = 2;
    const int cols = n_warps * GD_COLS;
    const dim3 grid((E + cols - 1) / cols, H, n_requests);
    const bool vec = ((uintptr_t)x % 16) == 0 && (ld % 4) == 0 && (q_col % 4) == 0 && (k_col % 4) == 0 &&
                     (v_col % 4) == 0 && (D % 4) == 0 && (E % 4) == 0;
    const int dp = (rl + GD_PAD) * GD_PARTS;
    const size_t smem = (size_t)(2 * ((2 * ch * dp + ch * cols + 2 * ch + 3) & ~3) + ch * cols + 3 * ch) * sizeof(float);
#define IB_GDSCAN(CH, RL, VEC)                                                                                     \
    do {                                                                                                           \
        if (smem > 48 * 1024) {                                                                                    \
            const int e = ib_allow_dynamic_smem(delta_scan_smem_set[VEC == 4], delta_scan_kernel<CH, RL, VEC>, 96 * 1024); \
            if (e != IB_OK) return e;                                                                              \
        }                                                                                                          \
        ib_launch(delta_scan_kernel<CH, RL, VEC>, grid, 32 * n_warps, smem, stream, x, ld, q_col, k_col, v_col, G, \
                  fade, fade_ld, beta, beta_ld, unit_eps, q_scale, state, slot_stride, q_start, slots, out, H, D, E); \
    } while (0)
#define IB_GDSCAN_RL(CH, VEC)                                                                                      \
    do {                                                                                                           \
        if (rl == 8) IB_GDSCAN(CH, 8, VEC); else if (rl == 16) IB_GDSCAN(CH, 16, VEC);                             \
        else if (rl == 32) IB_GDSCAN(CH, 32, VEC); else IB_GDSCAN(CH, 64, VEC);                                    \
    } while (0)
    if (ch == 1) { if (vec) IB_GDSCAN_RL(1, 4); else IB_GDSCAN_RL(1, 1); }
    else { if (vec) IB_GDSCAN_RL(16, 4); else IB_GDSCAN_RL(16, 1); }
#undef IB_GDSCAN_RL
#undef IB_GDSCAN
    return ib_launch_status();
}
