// Mixers with a matrix state per head that is carried from token to token:
//
//   mode 0, a decay per key channel (gated linear attention):
//       S_t = diag(a_t) S_{t-1} + k_t v_t^T,   o_t = S_t^T q_t,   a_t = sigmoid(z_t + b)^(1/tau)
//   mode 1, scalar gates with a running maximum (the matrix memory of xLSTM):
//       i_t = cap tanh((p_t + b_i) / cap),   f_t = logsigmoid(cap tanh((r_t + b_f) / cap))
//       m_t = max(f_t + m_{t-1}, i_t)
//       S_t = exp(f_t + m_{t-1} - m_t) S_{t-1} + exp(i_t - m_t) k_t v_t^T        (n_t the same with k_t alone)
//       o_t = S_t^T q_t / (max(|n_t . q_t|, exp(-m_t)) + 1e-6)
//   mode 2, a forget gate per key channel whose complement takes the key's place (HGRN2):
//       f_t = l + (1 - l) sigmoid(z_t + b),   S_t = diag(f_t) S_{t-1} + (1 - f_t) v_t^T,   o_t = S_t^T silu(q_t)
//       l is a lower bound per channel; there is no key: what the gate lets go is what the value fills
//
// S is [D, E] per head (D key channels, E value channels).  The state, the gates and every sum are float in both
// builds; q, k and v come from a projection in act_t.  A request's rows are walked in order, one token after the
// other, so a result does not depend on how the prompt was cut into steps or on what else the step holds.
//
// Work split: a block owns 32 columns of S for one (request, head); lane l owns column l, warp w the rows 16 w ..
// 16 w + 15, each lane's 16 numbers of S in registers.  Tokens go in chunks of 16: the block fetches the chunk's q, k,
// v and gates together, a chunk ahead (one trip to memory per chunk, under the walk of the chunk before), turns the gates into
// decays there with all threads (the exponentials, logarithms and hyperbolic tangents leave the sequential part;
// of the running maximum only a chain of additions and comparisons stays sequential), then every warp walks the
// chunk's tokens: per token 16 multiply-adds per lane for the update and 16 for the product with q, all operands but
// S and v read from shared memory as the same word for the whole warp.  The warps' partial products are summed
// through shared memory once per chunk.  In mode 1 the vector n is kept a row per lane by every warp for its rows,
// and n . q is a warp sum per token that does not stand in the way of the update.
//
// State of one slot, float: S as [H, D, E] (E contiguous: a warp's loads and stores are whole lines), then for
// mode 1 n as [H, D] and m as [H].
#include "common.cuh"

#define LS_CHUNK 16
#define LS_COLS 32

__device__ __forceinline__ float ls_logsigmoid(float z) { return fminf(z, 0.0f) - log1pf(expf(-fabsf(z))); }

#define LS_RW 16      // rows of S per warp
#define LS_TOK(CH) ((CH) > 1 ? (CH) / 2 : 1)   // tokens of a chunk that a thread fetches

// CH tokens per chunk: 16, or 1 for steps of single tokens (few registers, many blocks per SM).  MAXT: the most
// threads of a block, 256 (up to 128 key channels) or 512 (up to 256): the registers must allow that many.
// COLS columns of S per block: 32 (a lane per column), or 16 where a step has too few (request, head, 32 columns) to
// give every SM a block: the two halves of a warp then own the same 16 columns and eight rows each.
template <int MODE, int CH, int MAXT, int COLS>
__global__ void __launch_bounds__(MAXT)
linear_scan_kernel(const act_t* __restrict__ proj, long ld, int q_col, int k_col, int v_col,
                                   const float* __restrict__ gates, long ld_gates, const float* __restrict__ gate_bias,
                                   float gate_param, float q_scale, float* __restrict__ state, long slot_stride,
                                   const int* __restrict__ q_start, const int* __restrict__ slots,
                                   float* __restrict__ out, int H, int D, int E) {
    extern __shared__ __align__(16) float smem[];
    ib_grid_dependency_sync();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
    const int Dp = n_warps * LS_RW;                     // D rounded up: the rows beyond D hold zeros
    constexpr int HALVES = 32 / COLS, RL = LS_RW / HALVES;   // rows of S per lane
    const int col = lane % COLS, half_w = lane / COLS, n_units = n_warps * HALVES;
    const int h = blockIdx.y, r = blockIdx.z, e0 = blockIdx.x * COLS, d0 = warp * LS_RW, dl = d0 + half_w * RL;
    const int row0 = q_start[r], row1 = q_start[r + 1];
    if (row1 <= row0) return;                           // the whole block leaves
    float* q_s = smem;                                  // [CH][Dp]
    float* k_s = q_s + CH * Dp;                         // [CH][Dp]
    float* a_s = k_s + CH * Dp;                         // [CH][Dp]   mode 0: the decays
    float* v_s = a_s + (MODE != 1 ? CH * Dp : 0);       // [CH][COLS]
    float* part = v_s + CH * LS_COLS;                   // [CH][n_units][COLS]
    float* npart = part + CH * n_warps * LS_COLS;       // [CH][n_warps]     mode 1
    float* g_s = npart + CH * n_warps;                  // [3][CH]           mode 1: keep, take, exp(-m)
    float* m_s = g_s + 4 * CH;                          // [1]               mode 1: the running maximum

    float* st = state + (long)slots[r] * slot_stride;
    float* st_S = st + (long)h * D * E;
    float* st_n = st + (long)H * D * E + (long)h * D;
    float* st_m = st + (long)H * D * E + (long)H * D + h;
    const bool col_ok = e0 + col < E;

    // the state's loads carry no condition (see the chunk's loads below): the address is brought inside
    float S[RL];
    const int e_in = min(e0 + col, E - 1);
#pragma unroll
    for (int i = 0; i < RL; ++i) S[i] = st_S[(long)min(dl + i, D - 1) * E + e_in];
#pragma unroll
    for (int i = 0; i < RL; ++i) S[i] = (col_ok && dl + i < D) ? S[i] : 0.0f;
    const bool n_mine = lane < LS_RW && d0 + lane < D;  // mode 1: lanes 0..15 keep n of the rows d0 + lane
    float n_row = 0.0f;
    if (MODE == 1) {
        if (n_mine) n_row = st_n[d0 + lane];
        if (threadIdx.x == 0) *m_s = *st_m;
    }
    __syncthreads();

    // One chunk's inputs as every thread fetches them: the block has 2 Dp threads; thread (d, half) owns key channel
    // d of the chunk's tokens of that parity, and a share of the chunk's values.  They are asked for a chunk ahead and
    // wait in registers while the chunk before is walked, so a trip to memory is paid once and under cover.
    // Every load is issued whatever the chunk's length and the thread's channel (the address is brought inside the
    // request's rows and the head's channels; what does not count is dropped when the registers are used): loads
    // under a condition are waited for one by one, loads without one are all under way together.  The numbers stay
    // as they were stored (act_t) until they are used, so nothing waits for them before the chunk is walked.
    constexpr int NT = LS_TOK(CH);
    const int half = threadIdx.x >= Dp ? 1 : 0;
    const int d_mine = threadIdx.x - half * Dp;
    const bool d_ok = d_mine < D;
    const bool fetches = CH > 1 || half == 0;
    act_t rq[NT], rk[NT], rv[NT];
    float rg[NT], r_gi = 0.0f, r_gf = 0.0f;
    const float my_bias = (MODE != 1 && d_ok) ? gate_bias[h * D + d_mine] : 0.0f;
    const float my_low = (MODE == 2 && d_ok) ? gate_bias[H * D + h * D + d_mine] : 0.0f;      // mode 2: the lower bounds follow the biases
    const int d_in = d_ok ? d_mine : D - 1;
    const int last_row = row1 - 1;
    auto fetch = [&](int c0) {
#pragma unroll
        for (int i = 0; i < NT; ++i) {
            const int t = CH > 1 ? 2 * i + half : 0;
            const act_t* p = proj + (long)min(c0 + t, last_row) * ld;
            rq[i] = p[q_col + h * D + d_in];
            rk[i] = p[k_col + h * D + d_in];
            if (MODE != 1) rg[i] = gates[(long)min(c0 + t, last_row) * ld_gates + h * D + d_in];
            const int idx = threadIdx.x + i * blockDim.x;          // the values: [tokens][COLS columns]
            const int vt = min(idx / COLS, CH - 1), ve = min(e0 + (idx % COLS), E - 1);
            rv[i] = proj[(long)min(c0 + vt, last_row) * ld + v_col + h * E + ve];
        }
        if (MODE == 1 && warp == 0) {
            const float* gp = gates + (long)min(c0 + lane, last_row) * ld_gates;
            r_gi = gp[h];
            r_gf = gp[H + h];
        }
    };
    fetch(row0);

    for (int c0 = row0; c0 < row1; c0 += CH) {
        const int nc = min(CH, row1 - c0);
        // ---- the chunk's inputs from the registers to shared memory, gates turned into decays ---------------
#pragma unroll
        for (int i = 0; i < NT; ++i) {
            const int t = CH > 1 ? 2 * i + half : 0;
            if (t < nc && fetches) {
                if (MODE == 2) {
                    const float qv = ib_to_float(rq[i]);
                    const float f = my_low + (1.0f - my_low) / (1.0f + expf(-(rg[i] + my_bias)));
                    q_s[t * Dp + d_mine] = d_ok ? qv / (1.0f + expf(-qv)) * q_scale : 0.0f;
                    k_s[t * Dp + d_mine] = d_ok ? 1.0f - f : 0.0f;
                    a_s[t * Dp + d_mine] = d_ok ? f : 1.0f;
                } else {
                    q_s[t * Dp + d_mine] = d_ok ? ib_to_float(rq[i]) * q_scale : 0.0f;
                    k_s[t * Dp + d_mine] = d_ok ? ib_to_float(rk[i]) : 0.0f;
                    if (MODE == 0)
                        a_s[t * Dp + d_mine] = d_ok ? expf(ls_logsigmoid(rg[i] + my_bias) * gate_param) : 1.0f;   // 1 / tau
                }
            }
            const int idx = threadIdx.x + i * blockDim.x;
            if (idx < nc * COLS) v_s[idx] = (e0 + (idx % COLS) < E) ? ib_to_float(rv[i]) : 0.0f;
        }
        if (MODE == 1 && warp == 0) {
            const float cap = gate_param;
            float li = 0.0f, lf = 0.0f;
            if (lane < nc) {
                li = cap * tanhf((r_gi + gate_bias[h]) / cap);
                lf = ls_logsigmoid(cap * tanhf((r_gf + gate_bias[H + h]) / cap));
            }
            // the running maximum: the only chain over the chunk's tokens, additions and comparisons
            float m_prev = *m_s, m_before = 0.0f, m_mine = 0.0f;
            for (int t = 0; t < nc; ++t) {
                const float lit = __shfl_sync(0xffffffffu, li, t), lft = __shfl_sync(0xffffffffu, lf, t);
                const float m_new = fmaxf(lft + m_prev, lit);
                if (lane == t) { m_before = m_prev; m_mine = m_new; }
                m_prev = m_new;
            }
            __syncwarp();
            if (lane < nc) {
                g_s[lane] = expf(lf + m_before - m_mine);              // keep
                g_s[CH + lane] = expf(li - m_mine);                    // take
                g_s[2 * CH + lane] = expf(-m_mine);
            }
            if (lane == 0) *m_s = m_prev;
        }
        __syncthreads();
        if (c0 + CH < row1) fetch(c0 + CH);
        if (MODE == 1) {
            // n of this warp's rows over the chunk, and its products with q: the recurrence is one multiply-add a token,
            // the sixteen warp sums do not depend on one another and leave the walk below alone
            float pq[CH];
            const int dn = d0 + (lane & (LS_RW - 1));
#pragma unroll
            for (int t = 0; t < CH; ++t) {
                pq[t] = 0.0f;
                if (t < nc) {
                    n_row = n_mine ? fmaf(g_s[t], n_row, g_s[CH + t] * k_s[t * Dp + dn]) : 0.0f;
                    pq[t] = n_row * q_s[t * Dp + dn];
                }
            }
#pragma unroll
            for (int t = 0; t < CH; ++t) pq[t] = ib_warp_sum(pq[t]);
#pragma unroll
            for (int t = 0; t < CH; ++t)
                if (lane == t && t < nc) npart[t * n_warps + warp] = pq[t];
        }
        // ---- the tokens, one after the other ----------------------------------------------------------------
        for (int t = 0; t < nc; ++t) {
            const float vt = MODE == 1 ? v_s[t * COLS + col] * g_s[CH + t] : v_s[t * COLS + col];   // v times exp(i - m)
            const float4* q4 = reinterpret_cast<const float4*>(q_s + t * Dp + dl);
            const float4* k4 = reinterpret_cast<const float4*>(k_s + t * Dp + dl);
            const float4* a4 = reinterpret_cast<const float4*>(a_s + t * Dp + dl);
            const float keep = MODE == 1 ? g_s[t] : 0.0f;
            float acc0 = 0.0f, acc1 = 0.0f, acc2 = 0.0f, acc3 = 0.0f;
#pragma unroll
            for (int i = 0; i < RL / 4; ++i) {
                const float4 q = q4[i], k = k4[i];
                float4 a;
                if (MODE != 1) a = a4[i]; else a = make_float4(keep, keep, keep, keep);
                S[4 * i + 0] = fmaf(a.x, S[4 * i + 0], k.x * vt); acc0 = fmaf(S[4 * i + 0], q.x, acc0);
                S[4 * i + 1] = fmaf(a.y, S[4 * i + 1], k.y * vt); acc1 = fmaf(S[4 * i + 1], q.y, acc1);
                S[4 * i + 2] = fmaf(a.z, S[4 * i + 2], k.z * vt); acc2 = fmaf(S[4 * i + 2], q.z, acc2);
                S[4 * i + 3] = fmaf(a.w, S[4 * i + 3], k.w * vt); acc3 = fmaf(S[4 * i + 3], q.w, acc3);
            }
            part[(t * n_units + warp * HALVES + half_w) * COLS + col] = (acc0 + acc1) + (acc2 + acc3);
        }
        __syncthreads();
        // ---- the warps' shares of every token's product, summed ---------------------------------------------
        for (int idx = threadIdx.x; idx < nc * COLS; idx += blockDim.x) {
            const int t = idx / COLS, e = idx % COLS;
            float o = 0.0f;
            for (int u = 0; u < n_units; ++u) o += part[(t * n_units + u) * COLS + e];
            if (MODE == 1) {
                float nq = 0.0f;
                for (int w = 0; w < n_warps; ++w) nq += npart[t * n_warps + w];
                o /= fmaxf(fabsf(nq), g_s[2 * CH + t]) + 1e-6f;
            }
            if (e0 + e < E) out[((long)(c0 + t) * H + h) * E + e0 + e] = o;
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < RL; ++i)
        if (col_ok && dl + i < D) st_S[(long)(dl + i) * E + e0 + col] = S[i];
    if (MODE == 1 && blockIdx.x == 0) {
        if (n_mine) st_n[d0 + lane] = n_row;
        if (threadIdx.x == 0) *st_m = *m_s;
    }
}

static IbDeviceSet scan_smem_set[32];

// proj [rows, ld] act_t holds q and k as [H, D] and v as [H, E] from columns q_col, k_col, v_col on.
// gates [rows, ld_gates] float: mode 0 the decay's pre-activations [H, D] (gate_bias [H * D], gate_param = tau);
// mode 1 the input gate's and then the forget gate's pre-activations [2, H] (gate_bias [2 * H], gate_param = cap);
// mode 2 the forget gate's pre-activations [H, D] (gate_bias [2, H * D]: the biases and then the lower bounds; k_col is
// not read, gate_param is not used).
// out [rows, H, E] float.  state: see the head of the file; slot_stride floats per slot.  max_rows: the most rows
// that a request brings (1 chooses the form for steps of single tokens; any larger number the chunked form).
IB_EXPORT int ib_linear_scan(int mode, const void* proj, long ld, int q_col, int k_col, int v_col, const float* gates,
                             long ld_gates, const float* gate_bias, float gate_param, float q_scale, float* state,
                             long slot_stride, const int* q_start, const int* slots, int n_requests, float* out, int H,
                             int D, int E, int max_rows, cudaStream_t stream) {
    if (n_requests <= 0) return IB_OK;
    if (H <= 0 || D <= 0 || E <= 0 || proj == nullptr || gates == nullptr || gate_bias == nullptr || state == nullptr ||
        (mode < 0 || mode > 2) || !(gate_param > 0.0f))
        return IB_ERR_ARGUMENT;
    if (D > 256 || H > 65535 || n_requests > 65535) return IB_ERR_UNSUPPORTED;
    const long need = (long)H * E * D + (mode == 1 ? (long)H * D + H : 0);
    if (slot_stride < need) return IB_ERR_ARGUMENT;
    const int n_warps = D <= 16 ? 2 : (D + LS_RW - 1) / LS_RW;     // at least two: a thread per (channel, token parity)
    // 16 columns per block where 32 would leave most SMs without one (prompt portions of a few requests).  Measured
    // at 2,048 tokens of one request with 16 heads of 128 x 128: 0.48 against 0.62 ms with a decay per channel; with
    // scalar gates 0.96 against 0.72 ms (what a block does once per chunk for all its columns weighs more there), so
    // that mode keeps 32.
    const int cols = (mode != 1 && max_rows != 1 && (long)((E + LS_COLS - 1) / LS_COLS) * H * n_requests < 120) ? 16 : LS_COLS;
    const dim3 grid((E + cols - 1) / cols, H, n_requests);
    const float param = mode == 0 ? 1.0f / gate_param : gate_param;
    const int ch = max_rows == 1 ? 1 : LS_CHUNK;
    auto smem_for = [ch](int warps) {
        return (size_t)(3 * ch * warps * LS_RW + ch * LS_COLS + ch * warps * LS_COLS + ch * warps + 4 * ch + 4) * sizeof(float);
    };
    const size_t smem = smem_for(n_warps);
#define IB_SCAN_C(MODE, CH, MAXT, COLS, SET)                                                                         \
    do {                                                                                                             \
        if (smem > 48 * 1024) { /* the permission is given once per device, for the most that the kernel can ask */  \
            const int e = ib_allow_dynamic_smem(scan_smem_set[SET], linear_scan_kernel<MODE, CH, MAXT, COLS>, smem_for(16)); \
            if (e != IB_OK) return e;                                                                                \
        }                                                                                                            \
        ib_launch(linear_scan_kernel<MODE, CH, MAXT, COLS>, grid, 32 * n_warps, smem, stream, (const act_t*)proj, ld, \
                  q_col, k_col, v_col, gates, ld_gates, gate_bias, param, q_scale, state, slot_stride, q_start,      \
                  slots, out, H, D, E);                                                                              \
    } while (0)
#define IB_SCAN_T(MODE, CH, MAXT, SET)                                                                               \
    do {                                                                                                             \
        if (cols == 16 && CH > 1) IB_SCAN_C(MODE, LS_CHUNK, MAXT, 16, SET + 8); else IB_SCAN_C(MODE, CH, MAXT, 32, SET); \
    } while (0)
#define IB_SCAN(MODE, CH, SET)                                                                                       \
    do {                                                                                                             \
        if (32 * n_warps <= 256) IB_SCAN_T(MODE, CH, 256, SET); else IB_SCAN_T(MODE, CH, 512, SET + 4);              \
    } while (0)
    if (mode == 2 && ch == 1) IB_SCAN(2, 1, 16);
    else if (mode == 2) IB_SCAN(2, LS_CHUNK, 17);
    else if (mode == 0 && ch == 1) IB_SCAN(0, 1, 0);
    else if (mode == 0) IB_SCAN(0, LS_CHUNK, 1);
    else if (ch == 1) IB_SCAN(1, 1, 2);
    else IB_SCAN(1, LS_CHUNK, 3);
#undef IB_SCAN_C
#undef IB_SCAN_T
#undef IB_SCAN
    return ib_launch_status();
}
