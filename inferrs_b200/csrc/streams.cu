// A residual that is several streams wide, norms in groups, and the small kernels around mixers that keep
// their sums in 32-bit: embedding with learned positions, the update-read-norm step of hyper-connections,
// the per-head norm with an output gate, and the polynomial activation with unit-rms terms.
//
// The residual is float [rows, streams, width] in both builds; one stream is the ordinary residual.
#include "common.cuh"

#define IB_MAX_STREAMS 8
#define IB_MAX_GROUPS 64

// ---------------------------------------------------------------------------
// out[row, s, :] = table[ids[row], :] * scale + pos_table[positions[row], :]   for every stream s
// (pos_table may be absent).  The sum is formed in float32.
// ---------------------------------------------------------------------------
template <typename WT, typename PT>
__global__ void embedding_streams_kernel(const WT* __restrict__ table, const int* __restrict__ ids,
                                         const PT* __restrict__ pos_table, const int* __restrict__ positions,
                                         float* __restrict__ out, int width, int vocab, int max_pos, float scale,
                                         int streams) {
    ib_grid_dependency_sync();
    const int row = blockIdx.x;
    const int id = ids[row];
    const bool ok = id >= 0 && id < vocab;  // the host refuses such ids before the launch
    const WT* src = table + (size_t)(ok ? id : 0) * width;
    const PT* ps = nullptr;
    if (pos_table != nullptr) {
        const int p = positions[row];
        if (p >= 0 && p < max_pos) ps = pos_table + (size_t)p * width;
    }
    float* dst = out + (size_t)row * streams * width;
    for (int j = threadIdx.x; j < width; j += blockDim.x) {
        float v = ok ? ib_to_float(src[j]) * scale : 0.0f;
        if (ps) v += ib_to_float(ps[j]);
        for (int s = 0; s < streams; ++s) dst[(size_t)s * width + j] = v;
    }
}

IB_EXPORT int ib_embedding_streams(const void* table, int table_is_f32, const int* ids, const void* pos_table,
                                   int pos_is_f32, const int* positions, float* out, int n_rows, int width, int vocab,
                                   int max_pos, float scale, int streams, cudaStream_t stream) {
    if (n_rows <= 0) return IB_OK;
    if (width <= 0 || vocab <= 0 || streams <= 0 || (pos_table != nullptr && (positions == nullptr || max_pos <= 0)))
        return IB_ERR_ARGUMENT;
    const int threads = width >= 1024 ? 256 : 128;
#define IB_EMB(WT, PT)                                                                                        \
    ib_launch(embedding_streams_kernel<WT, PT>, n_rows, threads, 0, stream, (const WT*)table, ids,           \
              (const PT*)pos_table, positions, out, width, vocab, max_pos, scale, streams)
    if (table_is_f32 && pos_is_f32) IB_EMB(float, float);
    else if (table_is_f32) IB_EMB(float, __nv_bfloat16);
    else if (pos_is_f32) IB_EMB(__nv_bfloat16, float);
    else IB_EMB(__nv_bfloat16, __nv_bfloat16);
#undef IB_EMB
    return ib_launch_status();
}

// ---------------------------------------------------------------------------
// One row of the stream-wide residual x[s, :], s < S:
//   1. the sub-layer before left its output `delta` to be brought in:
//          x_t <- sum_s mix[s, t] x_s + gain[t] * delta        (all t at once from the old x; written back)
//      (no mix: x_t <- x_t + gain[t] * delta, gain absent: 1; no delta: nothing to do)
//   2. u = sum_t read[t] x_t                                    (read absent: the plain sum)
//   3. out = u, its `groups` equal consecutive parts each divided by sqrt(mean(part^2) + eps), times w.
// rows != nullptr : row rows[r] -> row r of out; nothing is written back (the last norm of a model).
// Everything in float32; only `out` is act_t.
// ---------------------------------------------------------------------------
struct alignas(sizeof(act_t) * 4) StreamVec4 { act_t v[4]; };

template <typename WT>
__global__ void stream_add_norm_kernel(float* __restrict__ residual, const act_t* __restrict__ delta,
                                       const float* __restrict__ mix, const float* __restrict__ gain,
                                       const float* __restrict__ read, const WT* __restrict__ weight,
                                       act_t* __restrict__ out, const int* __restrict__ rows, int streams, int width,
                                       int groups, float eps) {
    extern __shared__ __align__(16) float u_row[];          // [width]
    __shared__ float red[32];
    __shared__ float inv_g[IB_MAX_GROUPS];
    __shared__ float s_mix[IB_MAX_STREAMS * IB_MAX_STREAMS], s_gain[IB_MAX_STREAMS], s_read[IB_MAX_STREAMS];
    ib_grid_dependency_launch();
    const int S = streams;
    if (threadIdx.x < S * S) s_mix[threadIdx.x] = mix ? mix[threadIdx.x] : ((threadIdx.x / S == threadIdx.x % S) ? 1.0f : 0.0f);
    if (threadIdx.x < S) {
        s_gain[threadIdx.x] = gain ? gain[threadIdx.x] : 1.0f;
        s_read[threadIdx.x] = read ? read[threadIdx.x] : 1.0f;
    }
    ib_grid_dependency_wait();
    __syncthreads();
    const int r = blockIdx.x;
    const int src = rows ? rows[r] : r;
    float* res = residual + (size_t)src * S * width;
    const act_t* del = delta ? delta + (size_t)src * width : nullptr;
    const bool write_back = (rows == nullptr) && (del != nullptr);
    // Four columns a thread and step where the width allows it (16-byte loads of every stream); loads carry no
    // condition (a stream beyond the last is read as the last and dropped), so all of a step's loads are under way together.
    const bool vec = (width & 3) == 0 && (((uintptr_t)res | (uintptr_t)del | (uintptr_t)u_row) & 15) == 0;
    const int step = vec ? 4 : 1;
    for (int j = threadIdx.x * step; j < width; j += blockDim.x * step) {
        float x[IB_MAX_STREAMS][4], d[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
        for (int s = 0; s < IB_MAX_STREAMS; ++s) {
            const float* src = res + (size_t)min(s, S - 1) * width + j;
            if (vec) {
                const float4 v = *reinterpret_cast<const float4*>(src);
                x[s][0] = v.x; x[s][1] = v.y; x[s][2] = v.z; x[s][3] = v.w;
            } else {
                x[s][0] = *src; x[s][1] = x[s][2] = x[s][3] = 0.0f;
            }
        }
        if (del) {
            if (vec) {
                const StreamVec4 v = *reinterpret_cast<const StreamVec4*>(del + j);
#pragma unroll
                for (int c = 0; c < 4; ++c) d[c] = ib_to_float(v.v[c]);
            } else {
                d[0] = ib_to_float(del[j]);
            }
        }
        float u[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        if (del) {
#pragma unroll
            for (int t = 0; t < IB_MAX_STREAMS; ++t) {
                if (t < S) {
                    float v[4];
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        v[c] = 0.0f;
#pragma unroll
                        for (int s2 = 0; s2 < IB_MAX_STREAMS; ++s2)
                            if (s2 < S) v[c] = fmaf(s_mix[s2 * S + t], x[s2][c], v[c]);
                        v[c] = fmaf(s_gain[t], d[c], v[c]);
                        u[c] = fmaf(s_read[t], v[c], u[c]);
                    }
                    if (write_back) {
                        float* dst = res + (size_t)t * width + j;
                        if (vec) *reinterpret_cast<float4*>(dst) = make_float4(v[0], v[1], v[2], v[3]);
                        else *dst = v[0];
                    }
                }
            }
        } else {
#pragma unroll
            for (int t = 0; t < IB_MAX_STREAMS; ++t)
                if (t < S) {
#pragma unroll
                    for (int c = 0; c < 4; ++c) u[c] = fmaf(s_read[t], x[t][c], u[c]);
                }
        }
        if (vec) *reinterpret_cast<float4*>(u_row + j) = make_float4(u[0], u[1], u[2], u[3]);
        else u_row[j] = u[0];
    }
    __syncthreads();
    const int part = width / groups;
    for (int g = 0; g < groups; ++g) {
        float ss = 0.0f;
        for (int j = threadIdx.x; j < part; j += blockDim.x) {
            const float v = u_row[g * part + j];
            ss += v * v;
        }
        ss = ib_block_sum(ss, red);
        if (threadIdx.x == 0) inv_g[g] = 1.0f / sqrtf(ss / (float)part + eps);
    }
    __syncthreads();
    act_t* dst = out + (size_t)r * width;
    for (int j = threadIdx.x; j < width; j += blockDim.x)
        dst[j] = ib_from_float<act_t>(u_row[j] * inv_g[j / part] * ib_to_float(weight[j]));
}

static IbDeviceSet stream_norm_smem_f32, stream_norm_smem_bf16;

IB_EXPORT int ib_stream_add_norm(float* residual, const void* delta, const float* mix, const float* gain,
                                 const float* read, const void* weight, int weight_is_f32, void* out, const int* rows,
                                 int n_rows, int streams, int width, int groups, float eps, cudaStream_t stream) {
    if (n_rows <= 0) return IB_OK;
    if (width <= 0 || streams <= 0 || groups <= 0 || width % groups || weight == nullptr) return IB_ERR_ARGUMENT;
    if (streams > IB_MAX_STREAMS || groups > IB_MAX_GROUPS) return IB_ERR_UNSUPPORTED;
    const size_t smem = (size_t)width * sizeof(float);
    const size_t smem_most = 200 * 1024;      // the permission for more than 48 KB is given once per device, for the most
    if (smem > smem_most) return IB_ERR_UNSUPPORTED;
    const int threads = width >= 2048 ? 512 : (width >= 512 ? 256 : 128);
    if (weight_is_f32) {
        if (smem > 48 * 1024) {
            const int e = ib_allow_dynamic_smem(stream_norm_smem_f32, stream_add_norm_kernel<float>, smem_most);
            if (e != IB_OK) return e;
        }
        ib_launch(stream_add_norm_kernel<float>, n_rows, threads, smem, stream, residual, (const act_t*)delta, mix, gain,
                  read, (const float*)weight, (act_t*)out, rows, streams, width, groups, eps);
    } else {
        if (smem > 48 * 1024) {
            const int e = ib_allow_dynamic_smem(stream_norm_smem_bf16, stream_add_norm_kernel<__nv_bfloat16>, smem_most);
            if (e != IB_OK) return e;
        }
        ib_launch(stream_add_norm_kernel<__nv_bfloat16>, n_rows, threads, smem, stream, residual, (const act_t*)delta,
                  mix, gain, read, (const __nv_bfloat16*)weight, (act_t*)out, rows, streams, width, groups, eps);
    }
    return ib_launch_status();
}

// ---------------------------------------------------------------------------
// What stands between a mixer's heads and its output projection: per (row, head) an optional division by the
// root mean square over the head's values, an optional weight, and a gate taken from the same row of a
// projection:   out[row, h*E + e] = o[row, h, e] * inv_rms * w[...] * act(gate[row, h*E + e])
//   norm_mode   0: no norm; 1: divide by sqrt(mean(o^2) + eps)
//   w           absent, or [E] (w_per_head = 0: one weight for every head), or [H*E] (w_per_head = 1)
//   gate_act    0: silu, 1: sigmoid
//   o           float or act_t; element (row, h, e) at o[row * o_row + h * o_head + e], so that a head-major
//               [H, rows, E] result of a batched product is read in place
//   gate        act_t, row stride ld_gate (a slice of a wider projection)
// One warp per (row, head); 32-bit arithmetic.
// ---------------------------------------------------------------------------
template <typename OT, typename WT>
__global__ void head_norm_gate_kernel(const OT* __restrict__ o, long o_row, long o_head, const act_t* __restrict__ gate,
                                      long ld_gate, const WT* __restrict__ w, int w_per_head, int norm_mode,
                                      int gate_act, float eps, act_t* __restrict__ out, int n_rows, int heads, int e_dim) {
    ib_grid_dependency_sync();
    const int lane = threadIdx.x & 31;
    const long item = (long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (item >= (long)n_rows * heads) return;
    const int row = (int)(item / heads), h = (int)(item % heads);
    const OT* src = o + (long)row * o_row + (long)h * o_head;
    float inv = 1.0f;
    if (norm_mode) {
        float ss = 0.0f;
        for (int e = lane; e < e_dim; e += 32) {
            const float v = ib_to_float(src[e]);
            ss += v * v;
        }
        ss = ib_warp_sum(ss);
        inv = 1.0f / sqrtf(ss / (float)e_dim + eps);
    }
    const act_t* g = gate ? gate + (long)row * ld_gate + (long)h * e_dim : nullptr;     // no gate: the normed heads alone
    act_t* dst = out + ((long)row * heads + h) * e_dim;
    for (int e = lane; e < e_dim; e += 32) {
        float v = ib_to_float(src[e]) * inv;
        if (w) v *= ib_to_float(w[w_per_head ? h * e_dim + e : e]);
        if (g) {
            const float z = ib_to_float(g[e]);
            const float sg = 1.0f / (1.0f + expf(-z));
            v *= gate_act == 0 ? z * sg : sg;
        }
        dst[e] = ib_from_float<act_t>(v);
    }
}

// The same with a block of eight warps per (row, head), for heads of 512 numbers and more (one norm over all of a
// mixer's heads side by side, for instance): a warp alone would walk the row twice, 32 numbers at a time.
template <typename OT, typename WT>
__global__ void head_norm_gate_wide_kernel(const OT* __restrict__ o, long o_row, long o_head,
                                           const act_t* __restrict__ gate, long ld_gate, const WT* __restrict__ w,
                                           int w_per_head, int norm_mode, int gate_act, float eps,
                                           act_t* __restrict__ out, int heads, int e_dim) {
    __shared__ float red[32];
    ib_grid_dependency_sync();
    const int row = blockIdx.x / heads, h = blockIdx.x - row * heads;
    const OT* src = o + (long)row * o_row + (long)h * o_head;
    float inv = 1.0f;
    if (norm_mode) {
        float ss = 0.0f;
        for (int e = threadIdx.x; e < e_dim; e += blockDim.x) {
            const float v = ib_to_float(src[e]);
            ss += v * v;
        }
        ss = ib_block_sum(ss, red);
        inv = 1.0f / sqrtf(ss / (float)e_dim + eps);
    }
    const act_t* g = gate ? gate + (long)row * ld_gate + (long)h * e_dim : nullptr;
    act_t* dst = out + ((long)row * heads + h) * e_dim;
    for (int e = threadIdx.x; e < e_dim; e += blockDim.x) {
        float v = ib_to_float(src[e]) * inv;
        if (w) v *= ib_to_float(w[w_per_head ? h * e_dim + e : e]);
        if (g) {
            const float z = ib_to_float(g[e]);
            const float sg = 1.0f / (1.0f + expf(-z));
            v *= gate_act == 0 ? z * sg : sg;
        }
        dst[e] = ib_from_float<act_t>(v);
    }
}

IB_EXPORT int ib_head_norm_gate(const void* o, int o_is_f32, long o_row, long o_head, const void* gate, long ld_gate,
                                const void* w, int w_is_f32, int w_per_head, int norm_mode, int gate_act, float eps,
                                void* out, int n_rows, int heads, int e_dim, cudaStream_t stream) {
    if (n_rows <= 0) return IB_OK;
    if (heads <= 0 || e_dim <= 0 || gate_act < 0 || gate_act > 1) return IB_ERR_ARGUMENT;      // gate may be absent
    const int warps = 4;
    const long items = (long)n_rows * heads;
    if (e_dim >= 512 && items <= 0x7fffffffL) {
#define IB_HNGW(OT, WT)                                                                                        \
    ib_launch(head_norm_gate_wide_kernel<OT, WT>, dim3((unsigned)items), 256, 0, stream, (const OT*)o, o_row,  \
              o_head, (const act_t*)gate, ld_gate, (const WT*)w, w_per_head, norm_mode, gate_act, eps,         \
              (act_t*)out, heads, e_dim)
        if (o_is_f32) {
            if (w_is_f32) IB_HNGW(float, float); else IB_HNGW(float, __nv_bfloat16);
        } else {
            if (w_is_f32) IB_HNGW(act_t, float); else IB_HNGW(act_t, __nv_bfloat16);
        }
#undef IB_HNGW
        return ib_launch_status();
    }
    const dim3 grid((unsigned)((items + warps - 1) / warps));
#define IB_HNG(OT, WT)                                                                                         \
    ib_launch(head_norm_gate_kernel<OT, WT>, grid, 32 * warps, 0, stream, (const OT*)o, o_row, o_head,        \
              (const act_t*)gate, ld_gate, (const WT*)w, w_per_head, norm_mode, gate_act, eps, (act_t*)out,   \
              n_rows, heads, e_dim)
    if (o_is_f32) {
        if (w_is_f32) IB_HNG(float, float); else IB_HNG(float, __nv_bfloat16);
    } else {
        if (w_is_f32) IB_HNG(act_t, float); else IB_HNG(act_t, __nv_bfloat16);
    }
#undef IB_HNG
    return ib_launch_status();
}

// ---------------------------------------------------------------------------
// The polynomial activation with unit-rms terms, per row z of a feed-forward's inner size F:
//     out = a * z / r1 + b * z^2 / r2 + c * z^3 / r3 + e,     r_p = sqrt(mean((z^p)^2) + eps)
// coef = (a, b, c, e) in float32.  Powers element by element; sums in float32.
// ---------------------------------------------------------------------------
#define POLY_VEC (16 / (int)sizeof(act_t))      // elements per 16-byte load: 8 bfloat16 or 4 float
#define POLY_KEEP 4                             // loads that a thread keeps in registers between the two passes
struct alignas(16) PolyVec { act_t v[POLY_VEC]; };

template <bool VEC>
__global__ void poly_norm_kernel(const act_t* __restrict__ z, const float* __restrict__ coef, act_t* __restrict__ out,
                                 int width, float eps) {
    __shared__ float red[32];
    ib_grid_dependency_launch();
    const float a = coef[0], b = coef[1], c = coef[2], e = coef[3];
    ib_grid_dependency_wait();
    const act_t* src = z + (size_t)blockIdx.x * width;
    act_t* dst = out + (size_t)blockIdx.x * width;
    float s1 = 0.0f, s2 = 0.0f, s3 = 0.0f;
    if (VEC) {
        // the host picks a block that holds the row in POLY_KEEP loads per thread: the row is read once
        const int nv = width / POLY_VEC;
        const PolyVec* src_v = reinterpret_cast<const PolyVec*>(src);
        PolyVec keep[POLY_KEEP];
#pragma unroll
        for (int k = 0; k < POLY_KEEP; ++k) keep[k] = src_v[min((int)(threadIdx.x + k * blockDim.x), nv - 1)];
#pragma unroll
        for (int k = 0; k < POLY_KEEP; ++k) {
            if ((int)(threadIdx.x + k * blockDim.x) < nv) {
#pragma unroll
                for (int i = 0; i < POLY_VEC; ++i) {
                    const float v = ib_to_float(keep[k].v[i]);
                    const float v2 = v * v, v3 = v2 * v;
                    s1 += v2; s2 += v2 * v2; s3 += v3 * v3;
                }
            }
        }
        s1 = ib_block_sum(s1, red);
        s2 = ib_block_sum(s2, red);
        s3 = ib_block_sum(s3, red);
        const float k1 = a / sqrtf(s1 / (float)width + eps);
        const float k2 = b / sqrtf(s2 / (float)width + eps);
        const float k3 = c / sqrtf(s3 / (float)width + eps);
        PolyVec* dst_v = reinterpret_cast<PolyVec*>(dst);
#pragma unroll
        for (int k = 0; k < POLY_KEEP; ++k) {
            const int j = threadIdx.x + k * blockDim.x;
            if (j < nv) {
                PolyVec o;
#pragma unroll
                for (int i = 0; i < POLY_VEC; ++i) {
                    const float v = ib_to_float(keep[k].v[i]);
                    const float v2 = v * v;
                    o.v[i] = ib_from_float<act_t>(k1 * v + k2 * v2 + k3 * (v2 * v) + e);
                }
                dst_v[j] = o;
            }
        }
        return;
    }
    for (int j = threadIdx.x; j < width; j += blockDim.x) {
        const float v = ib_to_float(src[j]);
        const float v2 = v * v, v3 = v2 * v;
        s1 += v2;
        s2 += v2 * v2;
        s3 += v3 * v3;
    }
    s1 = ib_block_sum(s1, red);
    s2 = ib_block_sum(s2, red);
    s3 = ib_block_sum(s3, red);
    const float k1 = a / sqrtf(s1 / (float)width + eps);
    const float k2 = b / sqrtf(s2 / (float)width + eps);
    const float k3 = c / sqrtf(s3 / (float)width + eps);
    for (int j = threadIdx.x; j < width; j += blockDim.x) {
        const float v = ib_to_float(src[j]);
        const float v2 = v * v;
        dst[j] = ib_from_float<act_t>(k1 * v + k2 * v2 + k3 * (v2 * v) + e);
    }
}

IB_EXPORT int ib_poly_norm(const void* z, const float* coef, void* out, int n_rows, int width, float eps,
                           cudaStream_t stream) {
    if (n_rows <= 0) return IB_OK;
    if (width <= 0 || coef == nullptr) return IB_ERR_ARGUMENT;
    // 16-byte loads and the row in registers where the width is a multiple of a load and POLY_KEEP loads per thread
    // of a block of up to 1,024 threads hold it
    const int nv = width / POLY_VEC;
    if (width % POLY_VEC == 0 && nv <= POLY_KEEP * 1024 && (((uintptr_t)z | (uintptr_t)out) & 15) == 0) {
        int threads = 128;
        while (threads * POLY_KEEP < nv) threads <<= 1;
        ib_launch(poly_norm_kernel<true>, n_rows, threads, 0, stream, (const act_t*)z, coef, (act_t*)out, width, eps);
    } else {
        const int threads = width >= 4096 ? 512 : (width >= 1024 ? 256 : 128);
        ib_launch(poly_norm_kernel<false>, n_rows, threads, 0, stream, (const act_t*)z, coef, (act_t*)out, width, eps);
    }
    return ib_launch_status();
}

// ---------------------------------------------------------------------------
// Two slices of one projection's rows, each divided by its root mean square and multiplied by a weight:
//   the query latent  -> cq[row, :]                      (act_t, contiguous)
//   the key/value latent -> the request's cache page at the row's position (absent for a layer that reads
//                          another layer's latents)
// proj is act_t [rows, ld]; the slices start at columns q_col and kv_col.  One block per row.
// The cache plane is [n_pages, page_size, rank] act_t.
// ---------------------------------------------------------------------------
template <typename WT>
__global__ void latent_norm_store_kernel(const act_t* __restrict__ proj, long ld, int q_col, int q_rank,
                                         const WT* __restrict__ q_w, act_t* __restrict__ cq, int kv_col, int kv_rank,
                                         const WT* __restrict__ kv_w, act_t* __restrict__ plane,
                                         const int* __restrict__ block_table, int max_pages, int page_size, int n_pages,
                                         const int* __restrict__ row_request, const int* __restrict__ positions,
                                         float eps) {
    __shared__ float red[32];
    ib_grid_dependency_sync();
    const int row = blockIdx.x;
    const act_t* src = proj + (long)row * ld;
    {
        float ss = 0.0f;
        for (int j = threadIdx.x; j < q_rank; j += blockDim.x) {
            const float v = ib_to_float(src[q_col + j]);
            ss += v * v;
        }
        ss = ib_block_sum(ss, red);
        const float inv = 1.0f / sqrtf(ss / (float)q_rank + eps);
        for (int j = threadIdx.x; j < q_rank; j += blockDim.x)
            cq[(long)row * q_rank + j] = ib_from_float<act_t>(ib_to_float(src[q_col + j]) * inv * ib_to_float(q_w[j]));
    }
    if (plane != nullptr) {
        float ss = 0.0f;
        for (int j = threadIdx.x; j < kv_rank; j += blockDim.x) {
            const float v = ib_to_float(src[kv_col + j]);
            ss += v * v;
        }
        ss = ib_block_sum(ss, red);
        const float inv = 1.0f / sqrtf(ss / (float)kv_rank + eps);
        const int pos = positions[row];
        const int page = block_table[(long)row_request[row] * max_pages + pos / page_size];
        if (page >= 0 && page < n_pages) {          // a request that only pads a replayed step owns no pages
            act_t* dst = plane + ((long)page * page_size + pos % page_size) * kv_rank;
            for (int j = threadIdx.x; j < kv_rank; j += blockDim.x)
                dst[j] = ib_from_float<act_t>(ib_to_float(src[kv_col + j]) * inv * ib_to_float(kv_w[j]));
        }
    }
}

IB_EXPORT int ib_latent_norm_store(const void* proj, long ld, int q_col, int q_rank, const void* q_w, void* cq,
                                   int kv_col, int kv_rank, const void* kv_w, int w_is_f32, void* plane,
                                   const int* block_table, int max_pages, int page_size, int n_pages,
                                   const int* row_request, const int* positions, int n_rows, float eps,
                                   cudaStream_t stream) {
    if (n_rows <= 0) return IB_OK;
    if (q_rank <= 0 || q_w == nullptr || cq == nullptr) return IB_ERR_ARGUMENT;
    if (plane != nullptr && (kv_rank <= 0 || kv_w == nullptr || block_table == nullptr || page_size <= 0 ||
                             max_pages <= 0 || row_request == nullptr || positions == nullptr))
        return IB_ERR_ARGUMENT;
    const int widest = q_rank > kv_rank ? q_rank : kv_rank;
    const int threads = widest >= 1024 ? 256 : 128;
    if (w_is_f32)
        ib_launch(latent_norm_store_kernel<float>, n_rows, threads, 0, stream, (const act_t*)proj, ld, q_col, q_rank,
                  (const float*)q_w, (act_t*)cq, kv_col, kv_rank, (const float*)kv_w, (act_t*)plane, block_table,
                  max_pages, page_size, n_pages, row_request, positions, eps);
    else
        ib_launch(latent_norm_store_kernel<__nv_bfloat16>, n_rows, threads, 0, stream, (const act_t*)proj, ld, q_col,
                  q_rank, (const __nv_bfloat16*)q_w, (act_t*)cq, kv_col, kv_rank, (const __nv_bfloat16*)kv_w,
                  (act_t*)plane, block_table, max_pages, page_size, n_pages, row_request, positions, eps);
    return ib_launch_status();
}
