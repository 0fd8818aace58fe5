// Per-head and per-row pieces that stand between the matrix products of a layer:
//   - qkv_head_norm_store: biases, an RMS norm of every query and key head, rotation of part of a
//     head, q out, keys and values (of different widths) into the paged cache; the projection's
//     row may have further columns behind q, k and v (an output gate's, say),
//   - latent_store / latent_query / head_product: latent attention, where ONE normed vector c a
//     token stands for the keys and values of every head (k_h = Uk_h c, v_h = Uv_h c) and a short
//     rotated part is shared by all heads. The cache keeps [c | rotated part]; a query head is
//     carried into the latent space (q_h Uk_h), scores and weighted sums are taken there, and
//     head_product brings the sums back through Uv_h,
//   - gelu_tanh, token_gate (a small per-token table gated by a projection of the stream),
//     add_cast (pending update into the stream, and the stream in the run's type),
//     cols_cast (some columns of a projection in the run's type), head_norm_gate (an RMS norm of
//     every head times a sigmoid gate).
// All arithmetic is float32. A projection arrives as the S partial sums of a split matrix
// product, [S, rows, width], added in rising order of S wherever a value is read.
#include "common.cuh"
#include "mma_utils.cuh"

__device__ __forceinline__ float parts_sum(const float* p, int S, size_t stride) {
    float x = p[0];
    for (int s = 1; s < S; ++s) x += p[(size_t)s * stride];
    return x;
}
__device__ __forceinline__ float gelu_tanh_f(float z) {
    return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}
__device__ __forceinline__ float sigmoid_f(float z) { return 1.0f / (1.0f + expf(-z)); }

// ---------------------------------------------------------------- q/k/v heads: bias, norm, rotation, cache
// Row n of the projection: nq query heads of d, nkv key heads of d, nkv value heads of dv, then
// anything. One warp per (token, head).
#define HN_MAX_D 512
template <typename T>
__global__ void qkv_head_norm_store_kernel(const float* __restrict__ qkv, int S, size_t split_stride, int W,
                                           const float* __restrict__ bias, const float* __restrict__ qw,
                                           const float* __restrict__ kw, float eps, const float2* __restrict__ cs,
                                           int rot, const int* __restrict__ cache_pos, const int* __restrict__ tok_seq,
                                           const int* __restrict__ block_table, int bt_stride, T* __restrict__ q_out,
                                           T* __restrict__ kcache, T* __restrict__ vcache, int nq, int nkv, int d,
                                           int dv, int k_layout, int v_layout, int store_kv) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ __align__(16) float rowbuf[];   // [warps][max(d, dv)]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n = blockIdx.x;
    const int head = blockIdx.y * (blockDim.x >> 5) + warp;
    const int nheads = nq + (store_kv ? 2 * nkv : 0);
    if (head >= nheads) return;
    const bool is_q = head < nq, is_k = !is_q && head < nq + nkv;
    const int width = (is_q || is_k) ? d : dv;
    const int col = is_q ? head * d : (is_k ? nq * d + (head - nq) * d : nq * d + nkv * d + (head - nq - nkv) * dv);
    float* x = rowbuf + warp * max(d, dv);
    const float* src = qkv + (size_t)n * W + col;
    for (int e = lane; e < width; e += 32) x[e] = parts_sum(src + e, S, split_stride) + (bias ? bias[col + e] : 0.0f);
    __syncwarp();
    const float* nw = is_q ? qw : (is_k ? kw : nullptr);
    if (nw) {
        float ss = 0.0f;
        for (int e = lane; e < d; e += 32) ss += x[e] * x[e];
        ss = warp_sum(ss);
        const float r = 1.0f / sqrtf(ss / (float)d + eps);
        for (int e = lane; e < d; e += 32) x[e] = x[e] * r * nw[e];
        __syncwarp();
    }
    if ((is_q || is_k) && rot > 0) {
        const int half = rot >> 1;
        const float2* csn = cs + (size_t)n * half;
        for (int i = lane; i < half; i += 32) {
            const float2 c_s = csn[i];
            const float a = x[i], b = x[i + half];
            x[i] = a * c_s.x - b * c_s.y;
            x[i + half] = b * c_s.x + a * c_s.y;
        }
        __syncwarp();
    }
    if (is_q) {
        T* dst = q_out + ((size_t)n * nq + head) * d;
        for (int e = lane; e < d; e += 32) dst[e] = from_f32<T>(x[e]);
    } else {
        const int kvh = is_k ? head - nq : head - nq - nkv;
        const int cp = cache_pos[n];
        const int page = block_table[(size_t)tok_seq[n] * bt_stride + cp / LUMEN_PAGE];
        T* tile = (is_k ? kcache : vcache) + ((size_t)page * nkv + kvh) * LUMEN_PAGE * width;
        const int r = cp % LUMEN_PAGE, lay = is_k ? k_layout : v_layout;
        for (int e = lane; e < width; e += 32) tile[tile_offset(lay, r, e, width)] = from_f32<T>(x[e]);
    }
}

LUMEN_API int lumen_qkv_head_norm_store(const float* qkv, int n_split, long long split_stride, int W, const float* bias,
                                        const float* qw, const float* kw, float eps, const float* cs, int rot,
                                        const int* cache_pos, const int* tok_seq, const int* block_table, int bt_stride,
                                        void* q_out, void* kcache, void* vcache, int is_bf16, int N, int nq, int nkv,
                                        int d, int dv, int k_layout, int v_layout, int store_kv, cudaStream_t stream) {
    if (N <= 0) return 0;
    if (d <= 0 || d > HN_MAX_D || dv <= 0 || dv > HN_MAX_D || rot < 0 || rot > d || (rot & 1) || nq <= 0 || nkv < 0 ||
        n_split < 1 || W < nq * d + (store_kv ? nkv * (d + dv) : 0))
        return LUMEN_ERR_UNSUPPORTED;
    if (k_layout == LUMEN_LAYOUT_SW128 && (!is_bf16 || d % 64)) return LUMEN_ERR_UNSUPPORTED;
    if (v_layout == LUMEN_LAYOUT_SW128 && (!is_bf16 || dv % 64)) return LUMEN_ERR_UNSUPPORTED;
    const int warps = 4, nheads = nq + (store_kv ? 2 * nkv : 0);
    if ((nheads + warps - 1) / warps > 65535) return LUMEN_ERR_UNSUPPORTED;
    dim3 grid(N, (nheads + warps - 1) / warps);
    const size_t smem = (size_t)warps * (d > dv ? d : dv) * sizeof(float);
    if (is_bf16)
        lumen_launch(qkv_head_norm_store_kernel<__nv_bfloat16>, grid, dim3(warps * 32), smem, stream, qkv, n_split,
                     (size_t)split_stride, W, bias, qw, kw, eps, (const float2*)cs, rot, cache_pos, tok_seq, block_table,
                     bt_stride, (__nv_bfloat16*)q_out, (__nv_bfloat16*)kcache, (__nv_bfloat16*)vcache, nq, nkv, d, dv,
                     k_layout, v_layout, store_kv);
    else
        lumen_launch(qkv_head_norm_store_kernel<float>, grid, dim3(warps * 32), smem, stream, qkv, n_split,
                     (size_t)split_stride, W, bias, qw, kw, eps, (const float2*)cs, rot, cache_pos, tok_seq, block_table,
                     bt_stride, (float*)q_out, (float*)kcache, (float*)vcache, nq, nkv, d, dv, k_layout, v_layout,
                     store_kv);
    LUMEN_LAUNCH_CHECK();
    return 0;
}

// ---------------------------------------------------------------- latent attention: what the cache keeps
// Columns c0 .. c0 + R + r of the projection: the first R are RMS-normed (weight nw) and are the
// latent c, the last r are rotated over their first `rot` numbers; the cache row of the token
// receives [c | rotated part] (one "kv head" of width R + r, plain tiles). A block a token.
template <typename T>
__global__ void __launch_bounds__(128)
latent_store_kernel(const float* __restrict__ u, int S, size_t split_stride, int W, int c0, int R, int r,
                    const float* __restrict__ nw, float eps, const float2* __restrict__ cs, int rot,
                    const int* __restrict__ cache_pos, const int* __restrict__ tok_seq,
                    const int* __restrict__ block_table, int bt_stride, T* __restrict__ cache) {
    pdl_trigger();
    pdl_wait();
    __shared__ float red[32];
    const int n = blockIdx.x, tid = threadIdx.x;
    const float* src = u + (size_t)n * W + c0;
    const int cp = cache_pos[n];
    const int page = block_table[(size_t)tok_seq[n] * bt_stride + cp / LUMEN_PAGE];
    T* row = cache + ((size_t)page * LUMEN_PAGE + cp % LUMEN_PAGE) * (R + r);
    float ss = 0.0f;
    float keep[4];              // a latent of up to 512 stays in registers between the two passes
    int k = 0;
    for (int e = tid; e < R; e += 128, ++k) {
        const float x = parts_sum(src + e, S, split_stride);
        if (k < 4) keep[k] = x;
        ss += x * x;
    }
    ss = block_sum(ss, red);
    const float inv = 1.0f / sqrtf(ss / (float)R + eps);
    k = 0;
    for (int e = tid; e < R; e += 128, ++k)
        row[e] = from_f32<T>((k < 4 ? keep[k] : parts_sum(src + e, S, split_stride)) * inv * nw[e]);
    const int half = rot >> 1;
    const float2* csn = cs + (size_t)n * half;
    for (int i = tid; i < half; i += 128) {
        const float2 c_s = csn[i];
        const float a = parts_sum(src + R + i, S, split_stride), b = parts_sum(src + R + i + half, S, split_stride);
        row[R + i] = from_f32<T>(a * c_s.x - b * c_s.y);
        row[R + i + half] = from_f32<T>(b * c_s.x + a * c_s.y);
    }
    for (int e = rot + tid; e < r; e += 128) row[R + e] = from_f32<T>(parts_sum(src + R + e, S, split_stride));
}

LUMEN_API int lumen_latent_store(const float* u, int n_split, long long split_stride, int W, int c0, int R, int r,
                                 const float* nw, float eps, const float* cs, int rot, const int* cache_pos,
                                 const int* tok_seq, const int* block_table, int bt_stride, void* cache, int is_bf16,
                                 int N, cudaStream_t stream) {
    if (N <= 0) return 0;
    if (R <= 0 || r < 0 || rot < 0 || rot > r || (rot & 1) || c0 < 0 || c0 + R + r > W || n_split < 1)
        return LUMEN_ERR_UNSUPPORTED;
    if (is_bf16)
        lumen_launch(latent_store_kernel<__nv_bfloat16>, dim3(N), dim3(128), 0, stream, u, n_split, (size_t)split_stride,
                     W, c0, R, r, nw, eps, (const float2*)cs, rot, cache_pos, tok_seq, block_table, bt_stride,
                     (__nv_bfloat16*)cache);
    else
        lumen_launch(latent_store_kernel<float>, dim3(N), dim3(128), 0, stream, u, n_split, (size_t)split_stride, W, c0,
                     R, r, nw, eps, (const float2*)cs, rot, cache_pos, tok_seq, block_table, bt_stride, (float*)cache);
    LUMEN_LAUNCH_CHECK();
    return 0;
}

// ---------------------------------------------------------------- latent attention: the query in the latent space
// Row n of the query projection holds H heads of [d plain | r rotated]. out[n, h] =
// [ sum_j q[n, h, j] Uk[h d + j, :]  (R numbers) | the r rotated numbers ], float32 or bfloat16. Uk is
// stored [H d, R]. A block takes LQ_TOK tokens of one head and every gridDim.z-th run of 128 latent
// coordinates; a thread a latent coordinate. Block z = 0 also writes the rotated numbers.
#define LQ_TOK 8
template <typename TW, typename TO>
__global__ void __launch_bounds__(128)
latent_query_kernel(const float* __restrict__ q, int S, size_t split_stride, int W, const TW* __restrict__ uk, int H,
                    int d, int r, int R, const float2* __restrict__ cs, int rot, TO* __restrict__ out, int product,
                    int N) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ float qs[];          // [LQ_TOK][d]
    const int h = blockIdx.y, n0 = blockIdx.x * LQ_TOK, tid = threadIdx.x;
    const int nt = min(LQ_TOK, N - n0);
    if (product) for (int i = tid; i < LQ_TOK * d; i += 128) {
        const int t = i / d, j = i - t * d;
        qs[i] = t < nt ? parts_sum(q + (size_t)(n0 + t) * W + h * (d + r) + j, S, split_stride) : 0.0f;
    }
    __syncthreads();
    const TW* w = uk + (size_t)h * d * R;
    if (product) for (int e = blockIdx.z * 128 + tid; e < R; e += 128 * gridDim.z) {
        float acc[LQ_TOK];
#pragma unroll
        for (int t = 0; t < LQ_TOK; ++t) acc[t] = 0.0f;
        for (int j = 0; j < d; ++j) {
            const float wv = to_f32(w[(size_t)j * R + e]);
#pragma unroll
            for (int t = 0; t < LQ_TOK; ++t) acc[t] = fmaf(qs[t * d + j], wv, acc[t]);
        }
#pragma unroll
        for (int t = 0; t < LQ_TOK; ++t)
            if (t < nt) out[((size_t)(n0 + t) * H + h) * (R + r) + e] = from_f32<TO>(acc[t]);
    }
    if (blockIdx.z != 0) return;
    const int half = rot >> 1;
    for (int i = tid; i < nt * r; i += 128) {
        const int t = i / r, e = i - t * r;
        const float* src = q + (size_t)(n0 + t) * W + h * (d + r) + d;
        float x = parts_sum(src + e, S, split_stride);
        if (e < rot) {
            const int k = e < half ? e : e - half;
            const float2 c_s = cs[(size_t)(n0 + t) * half + k];
            const float other = parts_sum(src + (e < half ? e + half : e - half), S, split_stride);
            x = e < half ? x * c_s.x - other * c_s.y : x * c_s.x + other * c_s.y;
        }
        out[((size_t)(n0 + t) * H + h) * (R + r) + R + e] = from_f32<TO>(x);
    }
}

LUMEN_API int lumen_latent_query(const float* q, int n_split, long long split_stride, int W, const void* uk,
                                 int uk_is_bf16, int H, int d, int r, int R, const float* cs, int rot, void* out,
                                 int out_is_bf16, int product, int N, cudaStream_t stream) {
    if (N <= 0) return 0;
    if (H <= 0 || H > 65535 || d <= 0 || r < 0 || R <= 0 || rot < 0 || rot > r || (rot & 1) || W < H * (d + r) ||
        n_split < 1 || (size_t)LQ_TOK * d * sizeof(float) > 48 * 1024)
        return LUMEN_ERR_UNSUPPORTED;
    // product 0: the R numbers of every head are already there (lumen_head_gemm); only the rotated ones are made
    dim3 grid((N + LQ_TOK - 1) / LQ_TOK, H, product ? (R + 127) / 128 : 1);
    const size_t smem = (size_t)LQ_TOK * d * sizeof(float);
#define LQ_LAUNCH(TW, TO)                                                                                            \
    lumen_launch(latent_query_kernel<TW, TO>, grid, dim3(128), smem, stream, q, n_split, (size_t)split_stride, W,    \
                 (const TW*)uk, H, d, r, R, (const float2*)cs, rot, (TO*)out, product, N)
    if (uk_is_bf16 && out_is_bf16) LQ_LAUNCH(__nv_bfloat16, __nv_bfloat16);
    else if (uk_is_bf16) LQ_LAUNCH(__nv_bfloat16, float);
    else if (out_is_bf16) LQ_LAUNCH(float, __nv_bfloat16);
    else LQ_LAUNCH(float, float);
#undef LQ_LAUNCH
    LUMEN_LAUNCH_CHECK();
    return 0;
}

// An optional gate of one number a (token, head): the head's output is multiplied by
// sigmoid(gate[n, g0 + h]), gate float32 [S, N, W] partial sums; p null: no gate.
struct HeadGate {
    const float* p;
    int S;
    size_t split_stride;
    int W, g0;
    __device__ __forceinline__ float of(int n, int h) const {
        return p ? sigmoid_f(parts_sum(p + (size_t)n * W + g0 + h, S, split_stride)) : 1.0f;
    }
};

// ---------------------------------------------------------------- a product of its own for every head
// out[n, h, e] = sum_j x[n, h, j] w[h E + e, j]: x float32 [N, H, J], w [H E, J], out [N, H E] in
// the run's type. A block takes HP_TOK tokens of one head and every gridDim.z-th run of 8 output
// coordinates; a warp an output coordinate at a time, its lanes along j.
#define HP_TOK 8
template <typename TW, typename TO>
__global__ void __launch_bounds__(256)
head_product_kernel(const float* __restrict__ x, const TW* __restrict__ w, TO* __restrict__ out, int N, int H, int J,
                    int E, HeadGate hg) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ float xs[];          // [HP_TOK][J]
    const int h = blockIdx.y, n0 = blockIdx.x * HP_TOK, tid = threadIdx.x;
    const int nt = min(HP_TOK, N - n0);
    for (int i = tid; i < HP_TOK * J; i += 256) {
        const int t = i / J, j = i - t * J;
        xs[i] = t < nt ? x[((size_t)(n0 + t) * H + h) * J + j] : 0.0f;
    }
    __syncthreads();
    const int warp = tid >> 5, lane = tid & 31;
    for (int e = blockIdx.z * 8 + warp; e < E; e += 8 * gridDim.z) {
        const TW* wr = w + ((size_t)h * E + e) * J;
        float acc[HP_TOK];
#pragma unroll
        for (int t = 0; t < HP_TOK; ++t) acc[t] = 0.0f;
        for (int j = lane; j < J; j += 32) {
            const float wv = to_f32(wr[j]);
#pragma unroll
            for (int t = 0; t < HP_TOK; ++t) acc[t] = fmaf(xs[t * J + j], wv, acc[t]);
        }
#pragma unroll
        for (int t = 0; t < HP_TOK; ++t) acc[t] = warp_sum(acc[t]);
        if (lane == 0)
            for (int t = 0; t < nt; ++t) out[(size_t)(n0 + t) * H * E + h * E + e] = from_f32<TO>(acc[t] * hg.of(n0 + t, h));
    }
}

LUMEN_API int lumen_head_product(const float* x, const void* w, int w_is_bf16, void* out, int out_is_bf16, int N, int H,
                                 int J, int E, const float* gate, int gate_split, long long gate_split_stride,
                                 int gate_w, int gate_col, cudaStream_t stream) {
    if (N <= 0) return 0;
    if (gate && (gate_split < 1 || gate_col < 0 || gate_col + H > gate_w)) return LUMEN_ERR_BAD_ARGUMENT;
    const HeadGate hg = {gate, gate_split, (size_t)gate_split_stride, gate_w, gate_col};
    if (H <= 0 || H > 65535 || J <= 0 || E <= 0 || (size_t)HP_TOK * J * sizeof(float) > 48 * 1024)
        return LUMEN_ERR_UNSUPPORTED;
    // few tokens: a head's outputs are spread over more blocks, so that the step fills the device
    const int gz = N <= 8 * HP_TOK ? min(8, (E + 7) / 8) : 1;
    dim3 grid((N + HP_TOK - 1) / HP_TOK, H, gz);
    const size_t smem = (size_t)HP_TOK * J * sizeof(float);
    if (w_is_bf16 && out_is_bf16)
        lumen_launch(head_product_kernel<__nv_bfloat16, __nv_bfloat16>, grid, dim3(256), smem, stream, x,
                     (const __nv_bfloat16*)w, (__nv_bfloat16*)out, N, H, J, E, hg);
    else if (w_is_bf16)
        lumen_launch(head_product_kernel<__nv_bfloat16, float>, grid, dim3(256), smem, stream, x, (const __nv_bfloat16*)w,
                     (float*)out, N, H, J, E, hg);
    else if (out_is_bf16)
        lumen_launch(head_product_kernel<float, __nv_bfloat16>, grid, dim3(256), smem, stream, x, (const float*)w,
                     (__nv_bfloat16*)out, N, H, J, E, hg);
    else
        lumen_launch(head_product_kernel<float, float>, grid, dim3(256), smem, stream, x, (const float*)w, (float*)out, N, H, J, E, hg);
    LUMEN_LAUNCH_CHECK();
    return 0;
}

// ---------------------------------------------------------------- the same products on the tensor cores
// out[n, h, e] = sum_j x[n, h, j] B_h[j, e] for every head h, with x float32 (possibly partial sums,
// rounded to bfloat16 as it is staged), B_h bfloat16 and out bfloat16; mma.sync m16n8k16 with
// float32 accumulation. B_h is stored either [J][E] (B_KN: the keys' up-projection, whose rows are
// the plain query values) or [E][J] (the values' up-projection). A block takes 64 tokens and 128
// outputs of one head and walks j 32 at a time; the next step's operands are on their way to
// registers while this step's are multiplied. Row n of x starts at x + n xrs + h xhs, row n of out
// at out + n ors + h ohs.
#define HG_M 64
#define HG_N 128
#define HG_K 32
#define HG_LDA (HG_K + 8)
#define HG_LDB_KN (HG_N + 8)
template <bool B_KN>
__global__ void __launch_bounds__(128)
head_gemm_kernel(const float* __restrict__ x, int S, size_t split_stride, long long xrs, int xhs,
                 const __nv_bfloat16* __restrict__ w, int ldw, long long w_head_stride, __nv_bfloat16* __restrict__ out,
                 long long ors, int ohs, int N, int J, int E, HeadGate hg) {
    pdl_trigger();
    pdl_wait();
    __shared__ __align__(16) __nv_bfloat16 As[HG_M * HG_LDA];
    __shared__ __align__(16) __nv_bfloat16 Bs[B_KN ? HG_K * HG_LDB_KN : HG_N * HG_LDA];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n0 = blockIdx.x * HG_M, e0 = blockIdx.y * HG_N, h = blockIdx.z;
    const __nv_bfloat16* wh = w + (size_t)h * w_head_stride;

    // what this thread stages: 16 values of one row of x, and 32 values of one row of B
    const int ar = tid >> 1, ac = (tid & 1) * 16;
    const bool a_ok = n0 + ar < N;
    const float* xa = x + (size_t)(n0 + ar) * xrs + (size_t)h * xhs + ac;
    float4 pa[4];
    uint4 pb[4];
    auto fetch = [&](int k0) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            pa[i] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            if (a_ok) {
                pa[i] = *reinterpret_cast<const float4*>(xa + k0 + 4 * i);
                for (int sp = 1; sp < S; ++sp) {
                    const float4 v = *reinterpret_cast<const float4*>(xa + (size_t)sp * split_stride + k0 + 4 * i);
                    pa[i].x += v.x; pa[i].y += v.y; pa[i].z += v.z; pa[i].w += v.w;
                }
            }
        }
        if (B_KN) {         // row k0 + tid / 4 of B, 32 outputs from e0 + (tid % 4) * 32
            const int bk = tid >> 2, bc = e0 + (tid & 3) * 32;
#pragma unroll
            for (int i = 0; i < 4; ++i)
                pb[i] = (bc + 8 * i < E) ? *reinterpret_cast<const uint4*>(wh + (size_t)(k0 + bk) * ldw + bc + 8 * i)
                                         : make_uint4(0u, 0u, 0u, 0u);
        } else {            // row e0 + tid of B, its 32 values from k0
#pragma unroll
            for (int i = 0; i < 4; ++i)
                pb[i] = (e0 + tid < E) ? *reinterpret_cast<const uint4*>(wh + (size_t)(e0 + tid) * ldw + k0 + 8 * i)
                                       : make_uint4(0u, 0u, 0u, 0u);
        }
    };
    auto stage = [&]() {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            uint2 v;
            v.x = pack_bf16(pa[i].x, pa[i].y);
            v.y = pack_bf16(pa[i].z, pa[i].w);
            *reinterpret_cast<uint2*>(As + ar * HG_LDA + ac + 4 * i) = v;
        }
        if (B_KN) {
            const int bk = tid >> 2, bc = (tid & 3) * 32;
#pragma unroll
            for (int i = 0; i < 4; ++i) *reinterpret_cast<uint4*>(Bs + bk * HG_LDB_KN + bc + 8 * i) = pb[i];
        } else {
#pragma unroll
            for (int i = 0; i < 4; ++i) *reinterpret_cast<uint4*>(Bs + tid * HG_LDA + 8 * i) = pb[i];
        }
    };

    float acc[HG_N / 8][4];
#pragma unroll
    for (int i = 0; i < HG_N / 8; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.0f;
    const uint32_t a_addr = smem_u32(As) + (uint32_t)(((16 * warp + (lane & 7) + ((lane >> 3) & 1) * 8) * HG_LDA + (lane >> 4) * 8) * 2);
    const int mi = lane >> 3;
    const uint32_t b_addr = B_KN ? smem_u32(Bs) + (uint32_t)((((mi & 1) * 8 + (lane & 7)) * HG_LDB_KN + (mi >> 1) * 8) * 2)
                                 : smem_u32(Bs) + (uint32_t)((((lane & 7)) * HG_LDA + mi * 8) * 2);
    fetch(0);
    for (int k0 = 0; k0 < J; k0 += HG_K) {
        __syncthreads();            // the step before has been multiplied
        stage();
        __syncthreads();
        if (k0 + HG_K < J) fetch(k0 + HG_K);
        uint32_t a[2][4];
        ldsm_x4(a[0], a_addr);
        ldsm_x4(a[1], a_addr + 32);
        if (B_KN) {
#pragma unroll
            for (int np = 0; np < HG_N / 16; ++np)
#pragma unroll
                for (int kk = 0; kk < 2; ++kk) {
                    uint32_t r[4];
                    ldsm_x4_t(r, b_addr + (uint32_t)((16 * kk * HG_LDB_KN + 16 * np) * 2));
                    mma_bf16(acc[2 * np], a[kk], r[0], r[1]);
                    mma_bf16(acc[2 * np + 1], a[kk], r[2], r[3]);
                }
        } else {
#pragma unroll
            for (int nt = 0; nt < HG_N / 8; ++nt) {
                uint32_t r[4];
                ldsm_x4(r, b_addr + (uint32_t)(8 * nt * HG_LDA * 2));
                mma_bf16(acc[nt], a[0], r[0], r[1]);
                mma_bf16(acc[nt], a[1], r[2], r[3]);
            }
        }
    }
    const int g = lane >> 2, t = lane & 3;
    const int r0 = n0 + 16 * warp + g, r1 = r0 + 8;
    const float g0v = r0 < N ? hg.of(r0, h) : 1.0f, g1v = r1 < N ? hg.of(r1, h) : 1.0f;
#pragma unroll
    for (int nt = 0; nt < HG_N / 8; ++nt) {
        const int e = e0 + 8 * nt + 2 * t;
        if (e < E) {
            if (r0 < N) *reinterpret_cast<uint32_t*>(out + (size_t)r0 * ors + (size_t)h * ohs + e) = pack_bf16(acc[nt][0] * g0v, acc[nt][1] * g0v);
            if (r1 < N) *reinterpret_cast<uint32_t*>(out + (size_t)r1 * ors + (size_t)h * ohs + e) = pack_bf16(acc[nt][2] * g1v, acc[nt][3] * g1v);
        }
    }
}

// 1 if lumen_head_gemm takes these sizes: j in steps of 32, rows of x, B and out that keep 16-, 16-
// and 4-byte alignment.
LUMEN_API int lumen_head_gemm_takes(long long xrs, int xhs, long long split_stride, int ldw, long long w_head_stride,
                                    long long ors, int ohs, int J, int E) {
    return (J > 0 && J % HG_K == 0 && E > 0 && E % 8 == 0 && xrs % 4 == 0 && xhs % 4 == 0 && split_stride % 4 == 0 &&
            ldw % 8 == 0 && w_head_stride % 8 == 0 && ors % 2 == 0 && ohs % 2 == 0) ? 1 : 0;
}

// b_kn 1: B_h = w + h w_head_stride is [J][E] with rows ldw apart; 0: [E][J].
LUMEN_API int lumen_head_gemm(const float* x, int n_split, long long split_stride, long long xrs, int xhs, const void* w,
                              int b_kn, int ldw, long long w_head_stride, void* out, long long ors, int ohs, int N, int H,
                              int J, int E, const float* gate, int gate_split, long long gate_split_stride, int gate_w,
                              int gate_col, cudaStream_t stream) {
    if (N <= 0) return 0;
    if (gate && (gate_split < 1 || gate_col < 0 || gate_col + H > gate_w)) return LUMEN_ERR_BAD_ARGUMENT;
    const HeadGate hg = {gate, gate_split, (size_t)gate_split_stride, gate_w, gate_col};
    if (H <= 0 || H > 65535 || n_split < 1 || (E + HG_N - 1) / HG_N > 65535 ||
        !lumen_head_gemm_takes(xrs, xhs, split_stride, ldw, w_head_stride, ors, ohs, J, E))
        return LUMEN_ERR_UNSUPPORTED;
    dim3 grid((N + HG_M - 1) / HG_M, (E + HG_N - 1) / HG_N, H);
    if (b_kn)
        lumen_launch(head_gemm_kernel<true>, grid, dim3(128), 0, stream, x, n_split, (size_t)split_stride, xrs, xhs,
                     (const __nv_bfloat16*)w, ldw, w_head_stride, (__nv_bfloat16*)out, ors, ohs, N, J, E, hg);
    else
        lumen_launch(head_gemm_kernel<false>, grid, dim3(128), 0, stream, x, n_split, (size_t)split_stride, xrs, xhs,
                     (const __nv_bfloat16*)w, ldw, w_head_stride, (__nv_bfloat16*)out, ors, ohs, N, J, E, hg);
    LUMEN_LAUNCH_CHECK();
    return 0;
}

// ---------------------------------------------------------------- element-wise pieces
template <typename TO>
__global__ void gelu_tanh_kernel(const float* __restrict__ z, int S, size_t split_stride, TO* __restrict__ out,
                                 long long total) {
    pdl_trigger();
    pdl_wait();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x)
        out[i] = from_f32<TO>(gelu_tanh_f(parts_sum(z + i, S, split_stride)));
}

LUMEN_API int lumen_gelu_tanh(const float* z, int n_split, long long split_stride, void* out, int out_is_bf16,
                              long long total, cudaStream_t stream) {
    if (total <= 0) return 0;
    if (n_split < 1) return LUMEN_ERR_BAD_ARGUMENT;
    long long blocks = (total + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    if (out_is_bf16)
        lumen_launch(gelu_tanh_kernel<__nv_bfloat16>, dim3((int)blocks), dim3(256), 0, stream, z, n_split,
                     (size_t)split_stride, (__nv_bfloat16*)out, total);
    else
        lumen_launch(gelu_tanh_kernel<float>, dim3((int)blocks), dim3(256), 0, stream, z, n_split, (size_t)split_stride,
                     (float*)out, total);
    LUMEN_LAUNCH_CHECK();
    return 0;
}

// out[n, c] = gelu_tanh(z[n, c]) * table[tokens[n], col0 + c], c < C; z as partial sums [S, N, C].
template <typename TT, typename TO>
__global__ void token_gate_kernel(const float* __restrict__ z, int S, size_t split_stride, const int* __restrict__ tokens,
                                  const TT* __restrict__ table, int table_width, int col0, int C, TO* __restrict__ out,
                                  long long total) {
    pdl_trigger();
    pdl_wait();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const int n = (int)(i / C), c = (int)(i - (long long)n * C);
        const float e = to_f32(table[(size_t)tokens[n] * table_width + col0 + c]);
        out[i] = from_f32<TO>(gelu_tanh_f(parts_sum(z + i, S, split_stride)) * e);
    }
}

LUMEN_API int lumen_token_gate(const float* z, int n_split, long long split_stride, const int* tokens, const void* table,
                               int table_is_bf16, int table_width, int col0, int C, void* out, int out_is_bf16, int N,
                               cudaStream_t stream) {
    if (N <= 0) return 0;
    if (n_split < 1 || C <= 0 || col0 < 0 || col0 + C > table_width) return LUMEN_ERR_BAD_ARGUMENT;
    const long long total = (long long)N * C;
    long long blocks = (total + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
#define TG_LAUNCH(TT, TO)                                                                                              \
    lumen_launch(token_gate_kernel<TT, TO>, dim3((int)blocks), dim3(256), 0, stream, z, n_split, (size_t)split_stride, \
                 tokens, (const TT*)table, table_width, col0, C, (TO*)out, total)
    if (table_is_bf16 && out_is_bf16) TG_LAUNCH(__nv_bfloat16, __nv_bfloat16);
    else if (table_is_bf16) TG_LAUNCH(__nv_bfloat16, float);
    else if (out_is_bf16) TG_LAUNCH(float, __nv_bfloat16);
    else TG_LAUNCH(float, float);
#undef TG_LAUNCH
    LUMEN_LAUNCH_CHECK();
    return 0;
}

// h += sum of the partial sums of delta (when there are any); out = h in the run's type.
template <typename TO>
__global__ void add_cast_kernel(float* __restrict__ h, const float* __restrict__ delta, int S, size_t split_stride,
                                TO* __restrict__ out, long long total) {
    pdl_trigger();
    pdl_wait();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        float x = h[i];
        if (S > 0) {
            for (int s = 0; s < S; ++s) x += delta[(size_t)s * split_stride + i];
            h[i] = x;
        }
        out[i] = from_f32<TO>(x);
    }
}

LUMEN_API int lumen_add_cast(float* h, const float* delta, int n_split, long long split_stride, void* out,
                             int out_is_bf16, long long total, cudaStream_t stream) {
    if (total <= 0) return 0;
    if (n_split < 0) return LUMEN_ERR_BAD_ARGUMENT;
    long long blocks = (total + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    if (out_is_bf16)
        lumen_launch(add_cast_kernel<__nv_bfloat16>, dim3((int)blocks), dim3(256), 0, stream, h, delta, n_split,
                     (size_t)split_stride, (__nv_bfloat16*)out, total);
    else
        lumen_launch(add_cast_kernel<float>, dim3((int)blocks), dim3(256), 0, stream, h, delta, n_split,
                     (size_t)split_stride, (float*)out, total);
    LUMEN_LAUNCH_CHECK();
    return 0;
}

// out[n, c] = u[n, c0 + c] (its partial sums added), c < C, in the run's type.
template <typename TO>
__global__ void cols_cast_kernel(const float* __restrict__ u, int S, size_t split_stride, int W, int c0, int C,
                                 TO* __restrict__ out, long long total) {
    pdl_trigger();
    pdl_wait();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const long long n = i / C;
        const int c = (int)(i - n * C);
        out[i] = from_f32<TO>(parts_sum(u + n * W + c0 + c, S, split_stride));
    }
}

LUMEN_API int lumen_cols_cast(const float* u, int n_split, long long split_stride, int W, int c0, int C, void* out,
                              int out_is_bf16, int N, cudaStream_t stream) {
    if (N <= 0) return 0;
    if (n_split < 1 || C <= 0 || c0 < 0 || c0 + C > W) return LUMEN_ERR_BAD_ARGUMENT;
    const long long total = (long long)N * C;
    long long blocks = (total + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    if (out_is_bf16)
        lumen_launch(cols_cast_kernel<__nv_bfloat16>, dim3((int)blocks), dim3(256), 0, stream, u, n_split,
                     (size_t)split_stride, W, c0, C, (__nv_bfloat16*)out, total);
    else
        lumen_launch(cols_cast_kernel<float>, dim3((int)blocks), dim3(256), 0, stream, u, n_split, (size_t)split_stride,
                     W, c0, C, (float*)out, total);
    LUMEN_LAUNCH_CHECK();
    return 0;
}

// out[n, h, e] = y[n, h, e] / sqrt(mean_e(y[n, h, :]^2) + eps) * w[e] * sigmoid(gate[n, g0 + h E + e]);
// gate as partial sums [S, N, Wg]. One warp per (token, head).
template <typename TO>
__global__ void head_norm_gate_kernel(const float* __restrict__ y, const float* __restrict__ w, float eps,
                                      const float* __restrict__ gate, int S, size_t split_stride, int Wg, int g0,
                                      TO* __restrict__ out, int N, int H, int E) {
    pdl_trigger();
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + warp;
    if (item >= (long long)N * H) return;
    const int n = (int)(item / H), h = (int)(item - (long long)n * H);
    const float* src = y + (size_t)item * E;
    float ss = 0.0f;
    for (int e = lane; e < E; e += 32) ss += src[e] * src[e];
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)E + eps);
    for (int e = lane; e < E; e += 32) {
        const float g = parts_sum(gate + (size_t)n * Wg + g0 + h * E + e, S, split_stride);
        out[(size_t)item * E + e] = from_f32<TO>(src[e] * inv * w[e] * sigmoid_f(g));
    }
}

LUMEN_API int lumen_head_norm_gate(const float* y, const float* w, float eps, const float* gate, int n_split,
                                   long long split_stride, int Wg, int g0, void* out, int out_is_bf16, int N, int H,
                                   int E, cudaStream_t stream) {
    if (N <= 0) return 0;
    if (n_split < 1 || H <= 0 || E <= 0 || g0 < 0 || g0 + H * E > Wg) return LUMEN_ERR_BAD_ARGUMENT;
    const long long items = (long long)N * H;
    const int blocks = (int)((items + 7) / 8);
    if (out_is_bf16)
        lumen_launch(head_norm_gate_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, y, w, eps, gate, n_split,
                     (size_t)split_stride, Wg, g0, (__nv_bfloat16*)out, N, H, E);
    else
        lumen_launch(head_norm_gate_kernel<float>, dim3(blocks), dim3(256), 0, stream, y, w, eps, gate, n_split,
                     (size_t)split_stride, Wg, g0, (float*)out, N, H, E);
    LUMEN_LAUNCH_CHECK();
    return 0;
}

// ---------------------------------------------------------------- further element-wise pieces
// out = max(z, 0)^2; z as partial sums [S, total].
template <typename TO>
__global__ void relu2_kernel(const float* __restrict__ z, int S, size_t split_stride, TO* __restrict__ out,
                             long long total) {
    pdl_trigger();
    pdl_wait();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const float v = fmaxf(parts_sum(z + i, S, split_stride), 0.0f);
        out[i] = from_f32<TO>(v * v);
    }
}

LUMEN_API int lumen_relu2(const float* z, int n_split, long long split_stride, void* out, int out_is_bf16,
                          long long total, cudaStream_t stream) {
    if (total <= 0) return 0;
    if (n_split < 1) return LUMEN_ERR_BAD_ARGUMENT;
    long long blocks = (total + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    if (out_is_bf16)
        lumen_launch(relu2_kernel<__nv_bfloat16>, dim3((int)blocks), dim3(256), 0, stream, z, n_split,
                     (size_t)split_stride, (__nv_bfloat16*)out, total);
    else
        lumen_launch(relu2_kernel<float>, dim3((int)blocks), dim3(256), 0, stream, z, n_split, (size_t)split_stride,
                     (float*)out, total);
    LUMEN_LAUNCH_CHECK();
    return 0;
}

// A gated unit with clamped halves: row n of u (partial sums [S, N, W]) holds F gate values, then F
// up values; g = min(gate, limit), v = clamp(up, -limit, limit), out[n, f] = g sigmoid(alpha g) (v + 1),
// times sigmoid(u[n, tg]) when tg >= 0 (one gate a token, a further column of the same row).
__device__ __forceinline__ float clamped_glu_f(float g, float v, float limit, float alpha) {
    g = fminf(g, limit);
    v = fminf(fmaxf(v, -limit), limit);
    return g * sigmoid_f(alpha * g) * (v + 1.0f);
}
template <typename TO>
__global__ void clamped_glu_kernel(const float* __restrict__ u, int S, size_t split_stride, int W, int F, float limit,
                                   float alpha, int tg, TO* __restrict__ out, long long total) {
    pdl_trigger();
    pdl_wait();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const long long n = i / F;
        const int f = (int)(i - n * F);
        const float* row = u + n * W;
        float y = clamped_glu_f(parts_sum(row + f, S, split_stride), parts_sum(row + F + f, S, split_stride), limit, alpha);
        if (tg >= 0) y *= sigmoid_f(parts_sum(row + tg, S, split_stride));
        out[i] = from_f32<TO>(y);
    }
}

LUMEN_API int lumen_clamped_glu(const float* u, int n_split, long long split_stride, int W, int F, float limit,
                                float alpha, int token_gate_col, void* out, int out_is_bf16, int N,
                                cudaStream_t stream) {
    if (N <= 0) return 0;
    if (n_split < 1 || F <= 0 || 2 * F > W || token_gate_col >= W) return LUMEN_ERR_BAD_ARGUMENT;
    const long long total = (long long)N * F;
    long long blocks = (total + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    if (out_is_bf16)
        lumen_launch(clamped_glu_kernel<__nv_bfloat16>, dim3((int)blocks), dim3(256), 0, stream, u, n_split,
                     (size_t)split_stride, W, F, limit, alpha, token_gate_col, (__nv_bfloat16*)out, total);
    else
        lumen_launch(clamped_glu_kernel<float>, dim3((int)blocks), dim3(256), 0, stream, u, n_split,
                     (size_t)split_stride, W, F, limit, alpha, token_gate_col, (float*)out, total);
    LUMEN_LAUNCH_CHECK();
    return 0;
}

// out[n, c] = u[n, c0 + c] / sqrt(mean_c(u[n, c0 .. c0 + C]^2) + eps) * w[c]: an RMS norm of some
// columns of a projection (partial sums [S, N, W]), in the run's type; with a gate (partial sums [gS, N,
// gW]) also times sigmoid(gate[n, g0 + c]). A block a token.
template <typename TO>
__global__ void __launch_bounds__(1024)
cols_rmsnorm_kernel(const float* __restrict__ u, int S, size_t split_stride, int W, int c0, int C,
                    const float* __restrict__ w, float eps, TO* __restrict__ out, const float* __restrict__ gate, int gS,
                    size_t g_split_stride, int gW, int g0) {
    pdl_trigger();
    pdl_wait();
    __shared__ float red[32];
    const int n = blockIdx.x, nt = blockDim.x;
    const float* src = u + (size_t)n * W + c0;
    // a thread's values stay in registers where a row is at most 4 x the block wide
    float keep[4];
    float ss = 0.0f;
    int k = 0;
    for (int c = threadIdx.x; c < C; c += nt, ++k) {
        const float x = parts_sum(src + c, S, split_stride);
        if (k < 4) keep[k] = x;
        ss += x * x;
    }
    ss = block_sum(ss, red);
    const float inv = 1.0f / sqrtf(ss / (float)C + eps);
    k = 0;
    for (int c = threadIdx.x; c < C; c += nt, ++k) {
        const float x = k < 4 ? keep[k] : parts_sum(src + c, S, split_stride);
        float y = x * inv * w[c];
        if (gate) y *= sigmoid_f(parts_sum(gate + (size_t)n * gW + g0 + c, gS, g_split_stride));
        out[(size_t)n * C + c] = from_f32<TO>(y);
    }
}

LUMEN_API int lumen_cols_rmsnorm(const float* u, int n_split, long long split_stride, int W, int c0, int C,
                                 const float* w, float eps, void* out, int out_is_bf16, int N, const float* gate,
                                 int gate_split, long long gate_split_stride, int gate_w, int gate_col,
                                 cudaStream_t stream) {
    if (N <= 0) return 0;
    if (n_split < 1 || C <= 0 || c0 < 0 || c0 + C > W) return LUMEN_ERR_BAD_ARGUMENT;
    if (gate && (gate_split < 1 || gate_col < 0 || gate_col + C > gate_w)) return LUMEN_ERR_BAD_ARGUMENT;
    // few rows (decode steps): a row cannot fill the device, so its block is made wide and a thread's chain
    // of loads (a value's partial sums, one after the other) short
    int threads = 256;
    if (N < 2 * 148) {
        threads = ((C + 31) / 32) * 32;
        if (threads > 1024) threads = 1024;
        if (threads < 128) threads = 128;
    }
    if (out_is_bf16)
        lumen_launch(cols_rmsnorm_kernel<__nv_bfloat16>, dim3(N), dim3(threads), 0, stream, u, n_split, (size_t)split_stride,
                     W, c0, C, w, eps, (__nv_bfloat16*)out, gate, gate_split, (size_t)gate_split_stride, gate_w, gate_col);
    else
        lumen_launch(cols_rmsnorm_kernel<float>, dim3(N), dim3(threads), 0, stream, u, n_split, (size_t)split_stride, W, c0,
                     C, w, eps, (float*)out, gate, gate_split, (size_t)gate_split_stride, gate_w, gate_col);
    LUMEN_LAUNCH_CHECK();
    return 0;
}

// Logits in place: x <- x * scale, then, with cap > 0, x <- cap * tanh(x / cap).
__global__ void scale_softcap_kernel(float* __restrict__ x, float scale, float cap, long long total) {
    pdl_trigger();
    pdl_wait();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        float v = x[i] * scale;
        if (cap > 0.0f) v = cap * tanhf(v / cap);
        x[i] = v;
    }
}

LUMEN_API int lumen_scale_softcap(float* x, float scale, float cap, long long total, cudaStream_t stream) {
    if (total <= 0) return 0;
    long long blocks = (total + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    lumen_launch(scale_softcap_kernel, dim3((int)blocks), dim3(256), 0, stream, x, scale, cap, total);
    LUMEN_LAUNCH_CHECK();
    return 0;
}
