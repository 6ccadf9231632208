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
// lives in float.  A request's rows are walked in order by one block per (request, head, columns of S), so a result
// does not depend on what else the step holds, nor, beyond float rounding, on how the prompt was cut into steps.
//
// Two kernels: the first walks one token after the other (steps of one or two tokens per request); the second, further
// down, takes a prompt portion sixteen tokens at a time.
//
// Work split of the first: S^T k needs a whole column of S for every token, so a column is not cut over warps: a warp owns 8
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

// ---- the same rule over a chunk of sixteen tokens at once (prompt portions) ---------------------------------------------
//
// With F(a, b) = fade_a ... fade_b (1 where a > b), k' and q' the unit vectors, and S0 the state before the chunk's first
// token (token 0), the rule unrolls to
//     u_t  = beta_t (v_t - F(0, t) S0^T k'_t - sum_{j<t} F(j+1, t) (k'_j . k'_t) u_j)
//     o_t  = F(0, t) S0^T q'_t + sum_{j<=t} F(j+1, t) (k'_j . q'_t) u_j
//     S16  = F(0, 15) S0 + sum_j F(j+1, 15) k'_j u_j^T
// so that what is long (the products of S0 with the chunk's 32 vectors, the 120 + 136 dot products among them, the
// write of sixteen outer products) has no chain from token to token; what remains in order is a triangular
// substitution of sixteen short steps per column.  All of it is float, the sums in a fixed order.  F is made by
// multiplying the fades themselves, never by dividing, so a fade of zero stays a zero.
//
// A block of eight warps owns sixteen columns of S for one (request, head): lane & 15 is the column, the sixteen
// half-warps (units) own RL consecutive rows each, in registers.  Between two barriers: (1) every unit's share of
// S0^T q_t and S0^T k_t, and the tokens' unit factors (a warp per token); (2) the dot products among the chunk's
// vectors, two lanes per pair j < t, each with its F, and the units' shares summed;
// (3) the substitution, by every thread for its own column, then a token's read-out per unit, then the write.
// Tokens beyond a request's last one count as absent: their unit factors are zero, so nothing of what the buffer
// still holds from an earlier chunk enters a sum.
#define GC_CH 16
#define GC_COLS 16
#define GC_UNITS 16
#define GC_THREADS (32 * GC_UNITS / 2)
#define GC_PAIRS (GC_CH * (GC_CH - 1) / 2)
#define GC_PART_LD (GC_UNITS * GC_COLS + 16)    // a vector's partial sums, and sixteen floats so that two rows differ in banks
#define GC_EXTRA (2 * GC_CH * GC_PART_LD + 2 * GC_CH * GC_CH + 2 * GC_CH * GC_COLS + 4 * GC_CH + 4)

template <int RL, int VEC>
__global__ void __launch_bounds__(GC_THREADS, 2) delta_chunk_kernel(
    const float* __restrict__ x, long ld, int q_col, int k_col, int v_col, int G, const float* __restrict__ fade,
    long fade_ld, const float* __restrict__ beta, long beta_ld, float unit_eps, float q_scale,
    float* __restrict__ state, long slot_stride, const int* __restrict__ q_start, const int* __restrict__ slots,
    float* __restrict__ out, int H, int D, int E) {
    extern __shared__ __align__(16) float smem[];
    ib_grid_dependency_sync();
    // a row of q or k is followed by eight unused floats: rows that differ by one then differ by two banks of 16 bytes
    constexpr int CH = GC_CH, COLS = GC_COLS, Dp = GC_UNITS * RL + 8;
    constexpr int buf_floats = 2 * CH * Dp + CH * COLS + 2 * CH;  // q [CH][Dp], k [CH][Dp], v [CH][COLS], fade, beta
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int c = lane & (COLS - 1), unit = warp * 2 + (lane >> 4), dl = unit * RL;
    const int h = blockIdx.y, r = blockIdx.z, e0 = blockIdx.x * COLS;
    const int g = h / (H / G);
    const int row0 = q_start[r], row1 = q_start[r + 1];
    if (row1 <= row0) return;                                     // the whole block leaves
    float* part = smem + 2 * buf_floats;                          // [2 CH][GC_PART_LD] S0^T q_t, S0^T k_t by unit
    float* A_s = part + 2 * CH * GC_PART_LD;                      // [CH][CH] F(j+1, t) k'_j . k'_t, j < t
    float* B_s = A_s + CH * CH;                                   // [CH][CH] F(j+1, t) k'_j . q'_t, j <= t
    float* P_s = B_s + CH * CH;                                   // [2 CH][COLS] F(0, t) S0^T q'_t, then of k'_t
    float* qn_s = P_s + 2 * CH * COLS;                            // [CH] what makes q_t the unit vector, times q_scale
    float* kn_s = qn_s + CH;                                      // [CH] what makes k_t the unit vector
    float* kq_s = kn_s + CH;                                      // [CH] k_t . q_t as they were fetched
    float* w_s = kq_s + CH;                                       // [CH] F(t+1, 15) times k_t's factor; [CH]: F(0, 15)
    // what no copy or phase writes stays zero: rows beyond D, columns beyond E, A and B above their diagonals
    for (int i = threadIdx.x; i < 2 * buf_floats + GC_EXTRA; i += GC_THREADS) smem[i] = 0.0f;
    __syncthreads();

    float* st = state + (long)slots[r] * slot_stride + (long)h * D * E;
    const bool col_ok = e0 + c < E;
    float S[RL];
#pragma unroll
    for (int i = 0; i < RL; ++i) S[i] = (col_ok && dl + i < D) ? st[(long)(dl + i) * E + e0 + c] : 0.0f;
    const int e_n = min(COLS, E - e0);                            // this block's columns that exist

    auto fetch = [&](int c0, int buf) {
        const int nc = min(CH, row1 - c0);
        float* q_s = smem + buf * buf_floats;
        float* k_s = q_s + CH * Dp;
        float* v_s = k_s + CH * Dp;
        float* g_s = v_s + CH * COLS;
        if (VEC == 4) {
            const int d4 = D >> 2;
            for (int idx = threadIdx.x; idx < nc * d4; idx += GC_THREADS) {
                const int t = idx / d4, d = (idx - t * d4) << 2;
                const float* xr = x + (long)(c0 + t) * ld + g * D + d;
                gd_copy16(q_s + t * Dp + d, xr + q_col);
                gd_copy16(k_s + t * Dp + d, xr + k_col);
            }
            const int e4 = e_n >> 2;
            for (int idx = threadIdx.x; idx < nc * e4; idx += GC_THREADS) {
                const int t = idx / e4, e = (idx - t * e4) << 2;
                gd_copy16(v_s + t * COLS + e, x + (long)(c0 + t) * ld + v_col + h * E + e0 + e);
            }
        } else {
            for (int idx = threadIdx.x; idx < nc * D; idx += GC_THREADS) {
                const int t = idx / D, d = idx - t * D;
                const float* xr = x + (long)(c0 + t) * ld + g * D + d;
                gd_copy4(q_s + t * Dp + d, xr + q_col);
                gd_copy4(k_s + t * Dp + d, xr + k_col);
            }
            for (int idx = threadIdx.x; idx < nc * e_n; idx += GC_THREADS) {
                const int t = idx / e_n, e = idx - t * e_n;
                gd_copy4(v_s + t * COLS + e, x + (long)(c0 + t) * ld + v_col + h * E + e0 + e);
            }
        }
        if (threadIdx.x < nc) {
            gd_copy4(g_s + threadIdx.x, fade + (long)(c0 + threadIdx.x) * fade_ld + h);
            gd_copy4(g_s + CH + threadIdx.x, beta + (long)(c0 + threadIdx.x) * beta_ld + h);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    fetch(row0, 0);
    int pair_t = 1;                                               // this thread's pair j < t (the last sixteen: any)
    {
        const int p = min((int)(threadIdx.x >> 1), GC_PAIRS - 1);
        while ((pair_t + 1) * pair_t / 2 <= p) ++pair_t;
    }
    const int pair_j = min((int)(threadIdx.x >> 1), GC_PAIRS - 1) - pair_t * (pair_t - 1) / 2;

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
        const float* q_s = smem + buf * buf_floats;               // q's sixteen rows, then k's: 32 vectors in a row
        const float* k_s = q_s + CH * Dp;
        const float* v_s = k_s + CH * Dp;
        const float* g_s = v_s + CH * COLS;
        // ---- (1) S0^T times the 32 vectors, every unit its rows' share ----------------------------------------
#pragma unroll 8
        for (int v = 0; v < 2 * CH; ++v) {
            const float4* s4 = reinterpret_cast<const float4*>(q_s + v * Dp + dl);
            float a0 = 0.0f, a1 = 0.0f;
#pragma unroll
            for (int i = 0; i < RL / 4; ++i) {
                const float4 y = s4[i];
                a0 = fmaf(S[4 * i + 0], y.x, a0);
                a1 = fmaf(S[4 * i + 1], y.y, a1);
                a0 = fmaf(S[4 * i + 2], y.z, a0);
                a1 = fmaf(S[4 * i + 3], y.w, a1);
            }
            part[v * GC_PART_LD + unit * COLS + c] = a0 + a1;
        }
        // three numbers per token: the unit factors of q and k, and k . q (a warp per token)
        for (int t = warp; t < CH; t += GC_THREADS / 32) {
            float sq = 0.0f, sk = 0.0f, kq = 0.0f;
            for (int d = lane; d < D; d += 32) {
                const float a = q_s[t * Dp + d], b = k_s[t * Dp + d];
                sq = fmaf(a, a, sq);
                sk = fmaf(b, b, sk);
                kq = fmaf(a, b, kq);
            }
            sq = ib_warp_sum(sq);
            sk = ib_warp_sum(sk);
            kq = ib_warp_sum(kq);
            if (lane == 0) {
                const bool there = t < nc;
                qn_s[t] = !there ? 0.0f : (unit_eps >= 0.0f ? q_scale / sqrtf(sq + unit_eps) : q_scale);
                kn_s[t] = !there ? 0.0f : (unit_eps >= 0.0f ? 1.0f / sqrtf(sk + unit_eps) : 1.0f);
                kq_s[t] = there ? kq : 0.0f;
            }
        }
        __syncthreads();
        // ---- (2) the dot products among the chunk's vectors: two lanes per pair j < t, every other 16 bytes each
        auto F = [&](int a, int b) {          // fade_a ... fade_b over the tokens that exist, from four reads
            float f = 1.0f;
#pragma unroll
            for (int i4 = 0; i4 < CH / 4; ++i4) {
                const float4 y = reinterpret_cast<const float4*>(g_s)[i4];
                const int i = 4 * i4, hi = min(b, nc - 1);
                f *= (i + 0 >= a && i + 0 <= hi) ? y.x : 1.0f;
                f *= (i + 1 >= a && i + 1 <= hi) ? y.y : 1.0f;
                f *= (i + 2 >= a && i + 2 <= hi) ? y.z : 1.0f;
                f *= (i + 3 >= a && i + 3 <= hi) ? y.w : 1.0f;
            }
            return f;
        };
        {
            const int t = pair_t, j = pair_j, half = threadIdx.x & 1;
            const float4* kt4 = reinterpret_cast<const float4*>(k_s + t * Dp) + half;
            const float4* qt4 = reinterpret_cast<const float4*>(q_s + t * Dp) + half;
            const float4* kj4 = reinterpret_cast<const float4*>(k_s + j * Dp) + half;
            float kk0 = 0.0f, kk1 = 0.0f, qk0 = 0.0f, qk1 = 0.0f;
#pragma unroll 8
            for (int i = 0; i < GC_UNITS * RL / 4; i += 2) {
                const float4 a = kt4[i], b = qt4[i], y = kj4[i];
                kk0 = fmaf(a.x, y.x, kk0); kk1 = fmaf(a.y, y.y, kk1);
                kk0 = fmaf(a.z, y.z, kk0); kk1 = fmaf(a.w, y.w, kk1);
                qk0 = fmaf(b.x, y.x, qk0); qk1 = fmaf(b.y, y.y, qk1);
                qk0 = fmaf(b.z, y.z, qk0); qk1 = fmaf(b.w, y.w, qk1);
            }
            float kk = kk0 + kk1, qk = qk0 + qk1;
            kk += __shfl_xor_sync(0xffffffffu, kk, 1);
            qk += __shfl_xor_sync(0xffffffffu, qk, 1);
            if ((int)(threadIdx.x >> 1) < GC_PAIRS) {
                const float f = F(j + 1, t) * kn_s[j];
                if (half == 0) A_s[t * CH + j] = f * kn_s[t] * kk;
                else B_s[t * CH + j] = f * qn_s[t] * qk;
            } else {
                const int d = threadIdx.x - 2 * GC_PAIRS;         // the diagonal: a token's read-out sees its own write
                B_s[d * CH + d] = qn_s[d] * kn_s[d] * kq_s[d];
                w_s[d] = F(d + 1, CH - 1) * kn_s[d];
                if (d == 0) w_s[CH] = F(0, CH - 1);
            }
        }
        // the units' shares of S0^T q_t and S0^T k_t summed in a fixed order, with the token's factors
        const float gam_t = F(0, (threadIdx.x / COLS) & (CH - 1));     // both of a thread's sums are of one token
        for (int idx = threadIdx.x; idx < 2 * CH * COLS; idx += GC_THREADS) {
            const int v = idx / COLS, e = idx - v * COLS, t = v & (CH - 1);
            float s = 0.0f;
#pragma unroll
            for (int u = 0; u < GC_UNITS; ++u) s += part[v * GC_PART_LD + u * COLS + e];
            P_s[idx] = s * gam_t * (v < CH ? qn_s[t] : kn_s[t]);
        }
        __syncthreads();
        // ---- (3) the substitution, every thread for its own column --------------------------------------------
        float u_[CH];
#pragma unroll
        for (int t = 0; t < CH; ++t) {
            float acc = P_s[(CH + t) * COLS + c];
#pragma unroll
            for (int j4 = 0; j4 < (t + 3) / 4; ++j4) {
                const float4 a = reinterpret_cast<const float4*>(A_s + t * CH)[j4];
                if (4 * j4 + 0 < t) acc = fmaf(a.x, u_[4 * j4 + 0], acc);
                if (4 * j4 + 1 < t) acc = fmaf(a.y, u_[4 * j4 + 1], acc);
                if (4 * j4 + 2 < t) acc = fmaf(a.z, u_[4 * j4 + 2], acc);
                if (4 * j4 + 3 < t) acc = fmaf(a.w, u_[4 * j4 + 3], acc);
            }
            u_[t] = g_s[CH + t] * (v_s[t * COLS + c] - acc);
        }
        // a token's read-out per unit
        {
            const int t = unit;
            float o = P_s[t * COLS + c], o1 = 0.0f;
#pragma unroll
            for (int j4 = 0; j4 < CH / 4; ++j4) {
                const float4 b = reinterpret_cast<const float4*>(B_s + t * CH)[j4];
                o = fmaf(b.x, u_[4 * j4 + 0], o);
                o1 = fmaf(b.y, u_[4 * j4 + 1], o1);
                o = fmaf(b.z, u_[4 * j4 + 2], o);
                o1 = fmaf(b.w, u_[4 * j4 + 3], o1);
            }
            if (t < nc && col_ok) out[((long)(c0 + t) * H + h) * E + e0 + c] = o + o1;
        }
        // the state after the chunk
        const float keep = w_s[CH];
#pragma unroll
        for (int i = 0; i < RL; ++i) S[i] *= keep;
#pragma unroll
        for (int j = 0; j < CH; ++j) {
            const float uw = u_[j] * w_s[j];
            const float4* k4 = reinterpret_cast<const float4*>(k_s + j * Dp + dl);
#pragma unroll
            for (int i = 0; i < RL / 4; ++i) {
                const float4 y = k4[i];
                S[4 * i + 0] = fmaf(y.x, uw, S[4 * i + 0]);
                S[4 * i + 1] = fmaf(y.y, uw, S[4 * i + 1]);
                S[4 * i + 2] = fmaf(y.z, uw, S[4 * i + 2]);
                S[4 * i + 3] = fmaf(y.w, uw, S[4 * i + 3]);
            }
        }
        __syncthreads();       // before the next turn's copies and sums overwrite what this one read
    }
#pragma unroll
    for (int i = 0; i < RL; ++i)
        if (col_ok && dl + i < D) st[(long)(dl + i) * E + e0 + c] = S[i];
}

static IbDeviceSet delta_chunk_smem_set[8];
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
    const bool vec = ((uintptr_t)x % 16) == 0 && (ld % 4) == 0 && (q_col % 4) == 0 && (k_col % 4) == 0 &&
                     (v_col % 4) == 0 && (D % 4) == 0 && (E % 4) == 0;
    if (max_rows <= 0 || max_rows > 2) {       // prompt portions: sixteen tokens at once; one or two tokens cost less one by one
        const int crl = D <= 4 * GC_UNITS ? 4 : (D <= 8 * GC_UNITS ? 8 : 16);
        const int cdp = GC_UNITS * crl + 8;
        const size_t csmem = (size_t)(2 * (2 * GC_CH * cdp + GC_CH * GC_COLS + 2 * GC_CH) + GC_EXTRA) * sizeof(float);
        const dim3 cgrid((E + GC_COLS - 1) / GC_COLS, H, n_requests);
#define IB_GDCHUNK(RL, VEC, SET)                                                                                   \
    do {                                                                                                           \
        if (csmem > 48 * 1024) {                                                                                   \
            const int e = ib_allow_dynamic_smem(delta_chunk_smem_set[SET], delta_chunk_kernel<RL, VEC>, 128 * 1024); \
            if (e != IB_OK) return e;                                                                              \
        }                                                                                                          \
        ib_launch(delta_chunk_kernel<RL, VEC>, cgrid, GC_THREADS, csmem, stream, x, ld, q_col, k_col, v_col, G, fade,     \
                  fade_ld, beta, beta_ld, unit_eps, q_scale, state, slot_stride, q_start, slots, out, H, D, E);    \
    } while (0)
        if (crl == 4) { if (vec) IB_GDCHUNK(4, 4, 0); else IB_GDCHUNK(4, 1, 1); }
        else if (crl == 8) { if (vec) IB_GDCHUNK(8, 4, 2); else IB_GDCHUNK(8, 1, 3); }
        else { if (vec) IB_GDCHUNK(16, 4, 4); else IB_GDCHUNK(16, 1, 5); }
#undef IB_GDCHUNK
        return ib_launch_status();
    }
    const int ch = max_rows == 1 ? 1 : 16;
    const int rl = D <= 8 * GD_PARTS ? 8 : (D <= 16 * GD_PARTS ? 16 : (D <= 32 * GD_PARTS ? 32 : 64));
    // two warps (16 columns) per block where four would leave most SMs without a block
    int n_warps = (E + GD_COLS - 1) / GD_COLS;
    if (n_warps > 4) n_warps = 4;
    if (n_warps == 4 && ch > 1 && (long)((E + 31) / 32) * H * n_requests < 120) n_warps = 2;
    const int cols = n_warps * GD_COLS;
    const dim3 grid((E + cols - 1) / cols, H, n_requests);
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
