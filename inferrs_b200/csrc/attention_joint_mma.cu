// Paged attention whose heads' scores are mixed before the softmax and penalised by distance, on the tensor cores
// (bfloat16 in, float32 scores, softmax and accumulation).
//
// The mixing of scores across heads is linear, so it has been done on the queries before this kernel runs: a query
// head holds one vector per key/value head side by side (C * D numbers, C key/value heads), and its score against a
// token is the sum of its products with all C key heads of the token:
//
//     s[h, j] = scale * sum_c q~[h, c, :] . k[j, c, :]  -  bias[h, pos - j]
//
// bias [H, L] float is the distance penalty mixed the same way (a distance beyond the table reads its last entry; no
// table: no penalty).  Values are those of the head's own key/value head.
//
// One CTA works on one key/value head c0 of one tile of query rows: the rows are (token, head of group c0), so the
// values are read once for the group's heads; the keys of all C heads are read by every one of the C CTAs of a tile
// (they meet in L2).  Keys are walked in tiles of 64 (whole pages) brought in with cp.async, two tiles in flight; a
// key tile is C planes of [64, D], the value tile one.  The score of a tile is accumulated over the C planes by C
// times D / 16 steps of mma.sync, the queries' fragments coming from shared memory once per (plane, step).
//
// Two forms of the same loop, as in the plain tensor-core kernel:
//   prefill form : 128 rows (128 / Gq tokens of a prompt portion, Gq heads per key/value head); eight warps own 16
//                  rows each; two key tiles in shared memory where they fit beside the queries, else one.
//   decode form  : 16 rows (one token's Gq heads); the four warps take 16 keys each of every tile and the grid's z
//                  dimension splits the keys further; partial results go to scratch and a second kernel merges them.
// A row at position p sees keys lo..p of its request (ib_first_visible).
#include "common.cuh"

#if IB_ACT_BF16

#define JM_KEYS 64
#define JM_THREADS 128
#define JM_STAGES 2

__device__ __forceinline__ void jm_cp_async16(void* smem, const void* gmem, bool valid) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    const int bytes = valid ? 16 : 0;  // 0: the 16 bytes are filled with zeros
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(bytes));
}
__device__ __forceinline__ void jm_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void jm_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

__device__ __forceinline__ void jm_ldmatrix_x4(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3, const void* p) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(s));
}
__device__ __forceinline__ void jm_ldmatrix_x4_trans(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3,
                                                     const void* p) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(s));
}
__device__ __forceinline__ void jm_mma(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned jm_pack(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<unsigned*>(&v);
}
// element offset of 16-byte chunk `chunk` of row `row` in a [rows][D] tile whose chunks are XOR-swizzled
template <int D> __device__ __forceinline__ int jm_swz(int row, int chunk) {
    return row * D + ((chunk ^ (row & 7)) << 3);
}

struct JointMmaParams {
    const __nv_bfloat16* q;        // [N, n_heads, n_kv_heads * D]
    const __nv_bfloat16* k_pages;  // [n_pages, n_kv_heads, page_size, D]
    const __nv_bfloat16* v_pages;
    const int* block_table;        // [R, max_pages]
    const int* tile_req;           // [tiles] request of the tile
    const int* tile_row0;          // [tiles] first row (token) of the tile
    const int* q_start;            // [R + 1]
    const int* positions;          // [N]
    const float* bias;             // [n_heads, bias_len] or null
    __nv_bfloat16* out;            // [N, n_heads * D]
    float* part_o;                 // decode form with splits: [N, n_heads, splits, D]
    float* part_ml;                //                          [N, n_heads, splits, 2]
    int max_pages, page_size, n_pages, n_heads, n_kv_heads, window, n_splits, bias_len;
    float scale;
};

// PR: the rows of a prefill tile (a warp per 16 rows); the decode form has four warps on its 16 rows.
// ST: key tiles in shared memory, 2 (the next one on its way while this one is worked on) or 1.
template <int D, bool DECODE, int PR, int ST>
__global__ void __launch_bounds__(DECODE ? JM_THREADS : PR * 2) joint_attention_mma_kernel(const JointMmaParams P) {
    constexpr int ROWS = DECODE ? 16 : PR;
    constexpr int THREADS = DECODE ? JM_THREADS : PR * 2;
    constexpr int CH = D / 8;  // 16-byte chunks per row of a plane
    constexpr float LOG2E = 1.4426950408889634f;
    extern __shared__ __align__(128) unsigned char jm_smem[];
    const int C = P.n_kv_heads;
    __nv_bfloat16* sq = reinterpret_cast<__nv_bfloat16*>(jm_smem);     // [C][ROWS][D]
    __nv_bfloat16* sk = sq + C * ROWS * D;                             // [ST][C][64][D]
    __nv_bfloat16* sv = sk + ST * C * JM_KEYS * D;                     // [ST][64][D]

    ib_grid_dependency_sync();
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int gid = lane >> 2, tig = lane & 3;
    const int tile = blockIdx.x, kvh = blockIdx.y, split = blockIdx.z;
    const int req = P.tile_req[tile], row0 = P.tile_row0[tile];
    if (req < 0) return;                            // a place in a tile list of fixed length that holds no tile
    const int G = P.n_heads / C;                    // query heads per key/value head
    const int tpt = DECODE ? 1 : (ROWS / G);
    int n_tok = P.q_start[req + 1] - row0;
    if (n_tok > tpt) n_tok = tpt;
    const int p0 = P.positions[row0];
    const int pmax = p0 + n_tok - 1;
    const int lo_min = ib_first_visible(p0, P.window);
    const int t_first = lo_min / JM_KEYS, t_last = pmax / JM_KEYS + 1;
    int t_begin = t_first, t_end = t_last;
    if (DECODE && P.n_splits > 1) {
        const int per = (t_last - t_first + P.n_splits - 1) / P.n_splits;
        t_begin = t_first + split * per;
        t_end = t_begin + per < t_last ? t_begin + per : t_last;
    }
    const int* bt = P.block_table + (long)req * P.max_pages;
    const int dq = C * D;

    // queries of this tile: row r = (token r / G, head r % G of group kvh), plane by plane
    for (int idx = tid; idx < C * ROWS * CH; idx += THREADS) {
        const int c = idx / (ROWS * CH), rest = idx - c * (ROWS * CH);
        const int r = rest / CH, ch = rest - r * CH;
        const int ti = r / G, g = r - ti * G;
        const bool valid = ti < n_tok;
        const __nv_bfloat16* src = P.q + (((long)(row0 + (valid ? ti : 0)) * P.n_heads + kvh * G + g) * dq + c * D + ch * 8);
        jm_cp_async16(sq + c * ROWS * D + jm_swz<D>(r, ch), src, valid);
    }
    jm_commit();

    auto load_kv = [&](int t, int buf) {
        __nv_bfloat16* dk = sk + buf * C * JM_KEYS * D;
        __nv_bfloat16* dv = sv + buf * JM_KEYS * D;
        for (int idx = tid; idx < JM_KEYS * CH; idx += THREADS) {
            const int kk = idx / CH, ch = idx - kk * CH;
            const int j = t * JM_KEYS + kk;
            bool valid = j <= pmax && j >= lo_min;
            int page = 0;
            if (valid) {
                page = bt[j / P.page_size];
                valid = page >= 0 && page < P.n_pages;
            }
            const long slot = j % P.page_size;
            const int at = jm_swz<D>(kk, ch);
            for (int c = 0; c < C; ++c) {
                const long off = valid ? ((((long)page * C + c) * P.page_size + slot) * D + ch * 8) : 0;
                jm_cp_async16(dk + c * JM_KEYS * D + at, P.k_pages + off, valid);
                if (c == kvh) jm_cp_async16(dv + at, P.v_pages + off, valid);
            }
        }
    };

    // per-thread rows: ra = base + gid, rb = ra + 8
    const int rbase = DECODE ? 0 : warp * 16;
    int pos_r[2], lo_r[2];
    const float* bias_r[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int r = rbase + gid + 8 * h;
        const int ti = r / G, g = r - ti * G;
        bias_r[h] = P.bias ? P.bias + (long)(kvh * G + (g < G ? g : 0)) * P.bias_len : nullptr;
        if (ti < n_tok) {
            pos_r[h] = p0 + ti;
            lo_r[h] = ib_first_visible(pos_r[h], P.window);
        } else {
            pos_r[h] = -1;  // no key satisfies lo <= j <= pos
            lo_r[h] = 0;
        }
    }

    float o[D / 8][4];
#pragma unroll
    for (int n = 0; n < D / 8; ++n)
#pragma unroll
        for (int i = 0; i < 4; ++i) o[n][i] = 0.0f;
    float m_r[2] = {-INFINITY, -INFINITY}, l_r[2] = {0.0f, 0.0f};

#pragma unroll
    for (int i = 0; i < ST - 1; ++i) {
        if (t_begin + i < t_end) load_kv(t_begin + i, i);
        jm_commit();
    }

    constexpr int NP = DECODE ? 1 : 4;  // pairs of 8-key column tiles that this warp computes per key tile
    for (int t = t_begin; t < t_end; ++t) {
        const int buf = (t - t_begin) % ST;
        if (t + ST - 1 < t_end) load_kv(t + ST - 1, (t + ST - 1 - t_begin) % ST);  // the buffer of tile t - 1
        jm_commit();
        jm_wait<ST - 1>();      // the queries (first turn) and this tile's keys and values have landed
        __syncthreads();
        const __nv_bfloat16* tk = sk + buf * C * JM_KEYS * D;
        const __nv_bfloat16* tv = sv + buf * JM_KEYS * D;

        float s[2 * NP][4];
#pragma unroll
        for (int n = 0; n < 2 * NP; ++n)
#pragma unroll
            for (int i = 0; i < 4; ++i) s[n][i] = 0.0f;
        for (int c = 0; c < C; ++c) {
            const __nv_bfloat16* qc = sq + c * ROWS * D;
            const __nv_bfloat16* kc = tk + c * JM_KEYS * D;
#pragma unroll
            for (int ks = 0; ks < D / 16; ++ks) {
                unsigned qf[4];
                {
                    const int r = rbase + (lane & 7) + 8 * ((lane >> 3) & 1);
                    const int ch = 2 * ks + (lane >> 4);
                    jm_ldmatrix_x4(qf[0], qf[1], qf[2], qf[3], qc + jm_swz<D>(r, ch));
                }
#pragma unroll
                for (int np = 0; np < NP; ++np) {
                    const int key0 = DECODE ? warp * 16 : np * 16;
                    unsigned b0, b1, b2, b3;
                    const int kr = key0 + (lane & 7) + 8 * (lane >> 4);
                    const int ch = 2 * ks + ((lane >> 3) & 1);
                    jm_ldmatrix_x4(b0, b1, b2, b3, kc + jm_swz<D>(kr, ch));
                    jm_mma(s[2 * np], qf, b0, b1);
                    jm_mma(s[2 * np + 1], qf, b2, b3);
                }
            }
        }
        // scale, penalty, mask, running maximum (scores in units of log2 e from here on)
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int n = 0; n < 2 * NP; ++n) {
            const int col0 = (DECODE ? warp * 16 : 0) + n * 8 + 2 * tig;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int h = i >> 1;
                const int j = t * JM_KEYS + col0 + (i & 1);
                const bool vis = j >= lo_r[h] && j <= pos_r[h];
                float v = -INFINITY;
                if (vis) {
                    v = s[n][i] * P.scale;
                    if (bias_r[h]) {
                        const int dist = pos_r[h] - j;
                        v -= __ldg(bias_r[h] + (dist < P.bias_len ? dist : P.bias_len - 1));
                    }
                    v *= LOG2E;
                }
                s[n][i] = v;
                mx[h] = fmaxf(mx[h], v);
            }
        }
        float corr[2], msafe[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
            mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
            const float m_new = fmaxf(m_r[h], mx[h]);
            msafe[h] = m_new == -INFINITY ? 0.0f : m_new;
            corr[h] = m_r[h] == -INFINITY ? 0.0f : exp2f(m_r[h] - msafe[h]);
            m_r[h] = m_new;
            l_r[h] *= corr[h];
        }
#pragma unroll
        for (int n = 0; n < D / 8; ++n) {
            o[n][0] *= corr[0]; o[n][1] *= corr[0];
            o[n][2] *= corr[1]; o[n][3] *= corr[1];
        }
#pragma unroll
        for (int n = 0; n < 2 * NP; ++n)
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float p = exp2f(s[n][i] - msafe[i >> 1]);  // exp2(-inf) = 0 for masked keys
                s[n][i] = p;
                l_r[i >> 1] += p;
            }
        // O += P V
#pragma unroll
        for (int kt = 0; kt < NP; ++kt) {
            unsigned a[4];
            a[0] = jm_pack(s[2 * kt][0], s[2 * kt][1]);
            a[1] = jm_pack(s[2 * kt][2], s[2 * kt][3]);
            a[2] = jm_pack(s[2 * kt + 1][0], s[2 * kt + 1][1]);
            a[3] = jm_pack(s[2 * kt + 1][2], s[2 * kt + 1][3]);
            const int key0 = DECODE ? warp * 16 : kt * 16;
#pragma unroll
            for (int dn = 0; dn < D / 16; ++dn) {
                unsigned b0, b1, b2, b3;
                const int kr = key0 + (lane & 7) + 8 * ((lane >> 3) & 1);
                const int ch = 2 * dn + (lane >> 4);
                jm_ldmatrix_x4_trans(b0, b1, b2, b3, tv + jm_swz<D>(kr, ch));
                jm_mma(o[2 * dn], a, b0, b1);
                jm_mma(o[2 * dn + 1], a, b2, b3);
            }
        }
        __syncthreads();  // the next iteration's loads overwrite the other buffer, which all warps have left
    }
    jm_wait<0>();
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        l_r[h] += __shfl_xor_sync(0xffffffffu, l_r[h], 1);
        l_r[h] += __shfl_xor_sync(0xffffffffu, l_r[h], 2);
    }

    if (!DECODE) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int r = rbase + gid + 8 * h;
            const int ti = r / G, g = r - ti * G;
            if (ti >= n_tok) continue;
            const float inv = l_r[h] > 0.0f ? 1.0f / l_r[h] : 0.0f;
            __nv_bfloat16* dst = P.out + (((long)(row0 + ti) * P.n_heads + kvh * G + g) * D);
#pragma unroll
            for (int n = 0; n < D / 8; ++n) {
                const __nv_bfloat162 v = __floats2bfloat162_rn(o[n][2 * h] * inv, o[n][2 * h + 1] * inv);
                *reinterpret_cast<__nv_bfloat162*>(dst + n * 8 + 2 * tig) = v;
            }
        }
        return;
    }

    // decode form: the four warps hold partial results over different keys of the same 16 rows
    __syncthreads();
    float* so = reinterpret_cast<float*>(sk);            // [4 warps][16 rows][D]
    float* sm = so + 4 * 16 * D;                          // [4][16]
    float* sl = sm + 4 * 16;                              // [4][16]
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int r = gid + 8 * h;
        if (tig == 0) { sm[warp * 16 + r] = m_r[h]; sl[warp * 16 + r] = l_r[h]; }
#pragma unroll
        for (int n = 0; n < D / 8; ++n) {
            so[(warp * 16 + r) * D + n * 8 + 2 * tig] = o[n][2 * h];
            so[(warp * 16 + r) * D + n * 8 + 2 * tig + 1] = o[n][2 * h + 1];
        }
    }
    __syncthreads();
    for (int idx = tid; idx < G * D; idx += JM_THREADS) {
        const int g = idx / D, e = idx - g * D;  // row g of the tile is head g of the token's group
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; ++w) M = fmaxf(M, sm[w * 16 + g]);
        float acc = 0.0f, L = 0.0f;
        if (M > -INFINITY) {
#pragma unroll
            for (int w = 0; w < 4; ++w) {
                const float f = exp2f(sm[w * 16 + g] - M);
                acc += f * so[(w * 16 + g) * D + e];
                L += f * sl[w * 16 + g];
            }
        }
        const long head = (long)row0 * P.n_heads + kvh * G + g;
        if (P.n_splits > 1) {
            P.part_o[(head * P.n_splits + split) * D + e] = acc;
            if (e == 0) {
                P.part_ml[(head * P.n_splits + split) * 2] = M;
                P.part_ml[(head * P.n_splits + split) * 2 + 1] = L;
            }
        } else {
            P.out[head * D + e] = __float2bfloat16_rn(L > 0.0f ? acc / L : 0.0f);
        }
    }
}

// out[row, head, :] = sum_s 2^(m_s - M) o_s / sum_s 2^(m_s - M) l_s
__global__ void joint_attention_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                             __nv_bfloat16* __restrict__ out, int n_splits, int head_dim) {
    ib_grid_dependency_sync();
    const long head = blockIdx.x;  // row * n_heads + head
    const float* ml = part_ml + head * n_splits * 2;
    float M = -INFINITY;
    for (int s = 0; s < n_splits; ++s) M = fmaxf(M, ml[2 * s]);
    for (int e = threadIdx.x; e < head_dim; e += blockDim.x) {
        float acc = 0.0f, L = 0.0f;
        if (M > -INFINITY) {
            for (int s = 0; s < n_splits; ++s) {
                const float f = exp2f(ml[2 * s] - M);
                acc += f * part_o[(head * n_splits + s) * head_dim + e];
                L += f * ml[2 * s + 1];
            }
        }
        out[head * head_dim + e] = __float2bfloat16_rn(L > 0.0f ? acc / L : 0.0f);
    }
}

static size_t joint_mma_smem(int d, int c, bool decode, int prefill_rows = 64, int stages = JM_STAGES) {
    const int rows = decode ? 16 : prefill_rows;
    size_t bytes = (size_t)(c * rows * d + stages * (c + 1) * JM_KEYS * d) * sizeof(__nv_bfloat16);
    const size_t merge = (size_t)(4 * 16 * d + 2 * 4 * 16) * sizeof(float) + (size_t)c * rows * d * sizeof(__nv_bfloat16);
    return decode && merge > bytes ? merge : bytes;
}

// Rows of a prefill tile for these sizes: 128 where the queries of 128 rows and two key tiles fit into shared memory
// (twice the warps on an SM, every key tile fetched for twice the rows), else 64.
// A prefill tile is 128 rows on eight warps.  Where the joint queries of 128 rows leave no room for two key tiles
// (4 key heads of 128 numbers) one is kept: the fetch then waits for the tile before it to be done with, which costs
// less than tiles of 64 rows on four warps did (373 us against 524 us for a prompt of 2,048 with 16 heads).
#define JM_PREFILL_ROWS 128
static int joint_mma_prefill_stages(int d, int c) {
    return joint_mma_smem(d, c, false, JM_PREFILL_ROWS, 2) <= 224 * 1024 ? 2 : 1;
}

template <int D, bool DECODE, int PR, int ST>
static int launch_joint_mma(const JointMmaParams& P, int n_tiles, cudaStream_t stream) {
    const size_t smem = joint_mma_smem(D, P.n_kv_heads, DECODE, PR, ST);
    static IbDeviceSet configured;   // the attribute is kept per device; it is set to the most that any call may ask
    if (const int e = ib_allow_dynamic_smem(configured, joint_attention_mma_kernel<D, DECODE, PR, ST>, 224 * 1024)) return e;
    const dim3 grid(n_tiles, P.n_kv_heads, DECODE ? P.n_splits : 1);
    ib_launch(joint_attention_mma_kernel<D, DECODE, PR, ST>, grid, DECODE ? JM_THREADS : PR * 2, smem, stream, P);
    return ib_launch_status();
}

template <int D>
static int launch_joint_mma_prefill(const JointMmaParams& P, int n_tiles, cudaStream_t stream) {
    if (joint_mma_prefill_stages(D, P.n_kv_heads) == 2) return launch_joint_mma<D, false, JM_PREFILL_ROWS, 2>(P, n_tiles, stream);
    return launch_joint_mma<D, false, JM_PREFILL_ROWS, 1>(P, n_tiles, stream);
}

// The shared memory that a call of these sizes needs (0: sizes that the kernel does not take).
IB_EXPORT int ib_joint_attention_mma_smem(int n_heads, int n_kv_heads, int head_dim, int page_size, int decode_form) {
    if (n_heads <= 0 || n_kv_heads <= 0 || n_heads % n_kv_heads || page_size <= 0) return 0;
    if ((head_dim != 64 && head_dim != 128) || JM_KEYS % page_size || n_heads / n_kv_heads > 16) return 0;
    const size_t smem = decode_form ? joint_mma_smem(head_dim, n_kv_heads, true)
                                    : joint_mma_smem(head_dim, n_kv_heads, false, JM_PREFILL_ROWS,
                                                     joint_mma_prefill_stages(head_dim, n_kv_heads));
    return smem <= 224 * 1024 ? (int)smem : 0;
}

// The rows of a prefill tile for these sizes (0: sizes that the kernel does not take): a tile holds this many divided by
// (n_heads / n_kv_heads) tokens of one request.
IB_EXPORT int ib_joint_attention_mma_rows(int n_heads, int n_kv_heads, int head_dim, int page_size) {
    if (ib_joint_attention_mma_smem(n_heads, n_kv_heads, head_dim, page_size, 0) == 0) return 0;
    return JM_PREFILL_ROWS;
}

// q [n_rows, n_heads, n_kv_heads * head_dim] joint queries; bias [n_heads, bias_len] float or null.
// decode_form != 0: every tile is one token (n_tiles == rows of the step); n_splits >= 1 with scratch for > 1.
IB_EXPORT int ib_joint_attention_mma(const void* q, const void* k_pages, const void* v_pages, const int* block_table,
                                     int max_pages, int page_size, int n_pages, const int* tile_req,
                                     const int* tile_row0, int n_tiles, const int* q_start, const int* positions,
                                     int n_rows, int n_heads, int n_kv_heads, int head_dim, float scale, int window,
                                     const float* bias, int bias_len, void* out, int decode_form, int n_splits,
                                     float* part_o, float* part_ml, cudaStream_t stream) {
    if (n_tiles <= 0) return IB_OK;
    if (n_heads <= 0 || n_kv_heads <= 0 || n_heads % n_kv_heads || page_size <= 0 || max_pages <= 0 ||
        (bias != nullptr && bias_len <= 0))
        return IB_ERR_ARGUMENT;
    if (ib_joint_attention_mma_smem(n_heads, n_kv_heads, head_dim, page_size, decode_form) == 0) return IB_ERR_UNSUPPORTED;
    if (decode_form && n_splits > 1 && (part_o == nullptr || part_ml == nullptr)) return IB_ERR_ARGUMENT;
    JointMmaParams P;
    P.q = (const __nv_bfloat16*)q; P.k_pages = (const __nv_bfloat16*)k_pages; P.v_pages = (const __nv_bfloat16*)v_pages;
    P.block_table = block_table; P.tile_req = tile_req; P.tile_row0 = tile_row0; P.q_start = q_start;
    P.positions = positions; P.bias = bias; P.out = (__nv_bfloat16*)out; P.part_o = part_o; P.part_ml = part_ml;
    P.max_pages = max_pages; P.page_size = page_size; P.n_pages = n_pages; P.n_heads = n_heads;
    P.n_kv_heads = n_kv_heads; P.window = window; P.n_splits = decode_form ? (n_splits < 1 ? 1 : n_splits) : 1;
    P.bias_len = bias_len; P.scale = scale;
    int rc;
    if (head_dim == 64)
        rc = decode_form ? launch_joint_mma<64, true, 64, 2>(P, n_tiles, stream) : launch_joint_mma_prefill<64>(P, n_tiles, stream);
    else
        rc = decode_form ? launch_joint_mma<128, true, 64, 2>(P, n_tiles, stream) : launch_joint_mma_prefill<128>(P, n_tiles, stream);
    if (rc != IB_OK) return rc;
    if (decode_form && P.n_splits > 1) {
        ib_launch(joint_attention_merge_kernel, n_rows * n_heads, head_dim < 128 ? 64 : 128, 0, stream,
                  (const float*)part_o, (const float*)part_ml, (__nv_bfloat16*)out, P.n_splits, head_dim);
        return ib_launch_status();
    }
    return IB_OK;
}

#else  // the float32 build has no tensor-core attention: its attention is the generic kernel

IB_EXPORT int ib_joint_attention_mma_smem(int, int, int, int, int) { return 0; }
IB_EXPORT int ib_joint_attention_mma_rows(int, int, int, int) { return 0; }

IB_EXPORT int ib_joint_attention_mma(const void*, const void*, const void*, const int*, int, int, int, const int*,
                                     const int*, int, const int*, const int*, int, int, int, int, float, int,
                                     const float*, int, void*, int, int, float*, float*, cudaStream_t) {
    return IB_ERR_UNSUPPORTED;
}

#endif
