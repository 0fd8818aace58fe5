// General causal attention over the paged cache, for any number of new tokens
// per sequence (whole prompts and single decoded tokens alike), any key size and
// any value size up to 512 (the two may differ), any number of heads and groups,
// with an optional window. All arithmetic is float32 with the precise expf. It is the
// attention of the 32-bit path and the plain device reference of the faster
// bfloat16 kernels.
//
// Options, each a parameter: `chunk` > 0 limits a query's sight to the keys of its own run of
// `chunk` positions counted from the sequence's start; `softcap` > 0 replaces a score s by
// softcap * tanh(s / softcap); `sink` adds exp(0) to the softmax's denominator (a key of score 0
// that has no value); `v_in_k` takes a key's value from the first dv numbers of the key's own
// row (a latent cache, where keys and values are one vector); `gate` multiplies the output by
// sigmoid of some columns of a projection that arrives as partial sums. Queries and outputs
// may be float32 over a bfloat16 cache (TQ).
//
// One block per (query token, query head). Keys are walked in chunks of 128
// whose boundaries are multiples of 128 in absolute position, so the order of
// every sum depends only on the query's own position: the result for a token
// is the same bit for bit whether it came in a prompt, alone, or in any batch.
#include "common.cuh"

#define AG_THREADS 128
#define AG_ACC 4
#define AG_MAX_D (AG_ACC * AG_THREADS)   // widest value
#define AG_MAX_Q 1024       // widest key (a latent cache's keys are the latent and the rotated part)

struct AttnOptions {
    int chunk;            // 0: none
    float softcap;        // 0: none
    int sink;             // 1: the denominator has one more term exp(0)
    int v_in_k;           // 1: values are the first dv numbers of the key rows
    const float* gate;    // partial sums [gS][N][g_width]; columns g_col0 + head * dv + e
    int gS;
    long long g_split_stride;
    int g_width, g_col0;
};

template <typename T, typename TQ>
__global__ void __launch_bounds__(AG_THREADS)
attn_generic_kernel(const TQ* __restrict__ q, const T* __restrict__ kcache, const T* __restrict__ vcache,
                    const int* __restrict__ block_table, int bt_stride,
                    const int* __restrict__ tok_seq, const int* __restrict__ tok_pos,
                    TQ* __restrict__ out, int nq, int nkv, int d, int dv, int window, float scale,
                    int layout, int v_layout, AttnOptions opt) {
    pdl_wait();      // nothing of this kernel touches global memory before this
    pdl_trigger();
    __shared__ float qs[AG_MAX_Q];
    __shared__ float ps[AG_THREADS];
    __shared__ float red[32];
    const int head = blockIdx.y, n = blockIdx.x, tid = threadIdx.x;
    const int kvh = head / (nq / nkv);
    const int p = tok_pos[n];
    const int* bt = block_table + (size_t)tok_seq[n] * bt_stride;
    const TQ* qrow = q + ((size_t)n * nq + head) * d;
    for (int e = tid; e < d; e += AG_THREADS) qs[e] = to_f32(qrow[e]);
    __syncthreads();

    int lo = 0;
    if (window > 0 && p - window + 1 > 0) lo = p - window + 1;
    if (opt.chunk > 0) lo = max(lo, (p / opt.chunk) * opt.chunk);
    float m = opt.sink ? 0.0f : -INFINITY, l = opt.sink ? 1.0f : 0.0f;
    const int v_row = opt.v_in_k ? d : dv;        // numbers a value row lies apart from the next
    float acc[AG_ACC];               // dims tid, tid + 128, ...
#pragma unroll
    for (int i = 0; i < AG_ACC; ++i) acc[i] = 0.0f;

    for (int c = lo / AG_THREADS; c <= p / AG_THREADS; ++c) {
        const int j = c * AG_THREADS + tid;
        const bool valid = (j >= lo) && (j <= p);
        float s = -INFINITY;
        if (valid) {
            const int page = bt[j / LUMEN_PAGE];
            const T* ktile = kcache + ((size_t)page * nkv + kvh) * LUMEN_PAGE * d;
            const int r = j % LUMEN_PAGE;
            float dot = 0.0f;
            for (int e = 0; e < d; ++e) dot = fmaf(qs[e], to_f32(ktile[tile_offset(layout, r, e, d)]), dot);
            s = dot * scale;
            if (opt.softcap > 0.0f) s = opt.softcap * tanhf(s / opt.softcap);
        }
        const float cm = block_max(s, red);
        const float m_new = fmaxf(m, cm);
        const float pj = valid ? expf(s - m_new) : 0.0f;
        const float corr = (m == -INFINITY) ? 0.0f : expf(m - m_new);
        __syncthreads();
        ps[tid] = pj;
        const float csum = block_sum(pj, red);  // has a __syncthreads before reading ps below
        l = l * corr + csum;
#pragma unroll
        for (int i = 0; i < AG_ACC; ++i) acc[i] *= corr;
        __syncthreads();
        const int jbeg = max(c * AG_THREADS, lo), jend = min(c * AG_THREADS + AG_THREADS - 1, p);
        for (int jj = jbeg; jj <= jend; ++jj) {
            const int page = bt[jj / LUMEN_PAGE];
            const T* vtile = vcache + ((size_t)page * nkv + kvh) * LUMEN_PAGE * v_row;
            const int r = jj % LUMEN_PAGE;
            const float w = ps[jj - c * AG_THREADS];
#pragma unroll
            for (int i = 0; i < AG_ACC; ++i)
                if (tid + i * AG_THREADS < dv)
                    acc[i] = fmaf(w, to_f32(vtile[tile_offset(v_layout, r, tid + i * AG_THREADS, v_row)]), acc[i]);
        }
        m = m_new;
        __syncthreads();
    }
    TQ* orow = out + ((size_t)n * nq + head) * dv;
    const float inv = 1.0f / l;
#pragma unroll
    for (int i = 0; i < AG_ACC; ++i) {
        const int e = tid + i * AG_THREADS;
        if (e >= dv) break;
        float o = acc[i] * inv;
        if (opt.gate) {
            const float* g = opt.gate + (size_t)n * opt.g_width + opt.g_col0 + head * dv + e;
            float z = g[0];
            for (int s = 1; s < opt.gS; ++s) z += g[(size_t)s * opt.g_split_stride];
            o *= 1.0f / (1.0f + expf(-z));
        }
        orow[e] = from_f32<TQ>(o);
    }
}

static int attn_generic_launch(const void* q, int q_is_f32, const void* kcache, const void* vcache,
                               const int* block_table, int bt_stride, const int* tok_seq, const int* tok_pos,
                               void* out, int is_bf16, int N, int nq, int nkv, int d, int dv, int window,
                               float scale, int layout, int v_layout, AttnOptions opt, cudaStream_t stream) {
    if (N <= 0) return 0;
    if (d <= 0 || dv <= 0 || dv > AG_MAX_D || nq <= 0 || nkv <= 0 || nq % nkv != 0 || window < 0 || opt.chunk < 0)
        return LUMEN_ERR_UNSUPPORTED;
    if (d > AG_MAX_Q) return LUMEN_ERR_UNSUPPORTED;
    if (opt.v_in_k && (dv > d || v_layout != layout)) return LUMEN_ERR_BAD_ARGUMENT;
    if (nq > 65535) return LUMEN_ERR_UNSUPPORTED;
    if (layout == LUMEN_LAYOUT_SW128 && (!is_bf16 || d % 64 != 0)) return LUMEN_ERR_UNSUPPORTED;
    if (v_layout == LUMEN_LAYOUT_SW128 && (!is_bf16 || (opt.v_in_k ? d : dv) % 64 != 0)) return LUMEN_ERR_UNSUPPORTED;
    dim3 grid(N, nq);
    if (is_bf16 && !q_is_f32)
        lumen_launch(attn_generic_kernel<__nv_bfloat16, __nv_bfloat16>, dim3(grid), dim3(AG_THREADS), 0, stream,
            (const __nv_bfloat16*)q, (const __nv_bfloat16*)kcache, (const __nv_bfloat16*)vcache,
            block_table, bt_stride, tok_seq, tok_pos, (__nv_bfloat16*)out, nq, nkv, d, dv, window, scale,
            layout, v_layout, opt);
    else if (is_bf16)
        lumen_launch(attn_generic_kernel<__nv_bfloat16, float>, dim3(grid), dim3(AG_THREADS), 0, stream,
            (const float*)q, (const __nv_bfloat16*)kcache, (const __nv_bfloat16*)vcache,
            block_table, bt_stride, tok_seq, tok_pos, (float*)out, nq, nkv, d, dv, window, scale,
            layout, v_layout, opt);
    else
        lumen_launch(attn_generic_kernel<float, float>, dim3(grid), dim3(AG_THREADS), 0, stream,
            (const float*)q, (const float*)kcache, (const float*)vcache, block_table, bt_stride,
            tok_seq, tok_pos, (float*)out, nq, nkv, d, dv, window, scale, layout, v_layout, opt);
    LUMEN_LAUNCH_CHECK();
    return 0;
}

LUMEN_API int lumen_attn_generic(const void* q, const void* kcache, const void* vcache,
                                 const int* block_table, int bt_stride, const int* tok_seq,
                                 const int* tok_pos, void* out, int is_bf16, int N, int nq, int nkv,
                                 int d, int dv, int window, float scale, int layout, int v_layout,
                                 cudaStream_t stream) {
    AttnOptions opt = {};
    return attn_generic_launch(q, 0, kcache, vcache, block_table, bt_stride, tok_seq, tok_pos, out, is_bf16, N, nq,
                               nkv, d, dv, window, scale, layout, v_layout, opt, stream);
}

// The same with the options of AttnOptions; q_is_f32: queries and outputs are float32 whatever
// the cache's type.
LUMEN_API int lumen_attn_generic_opt(const void* q, int q_is_f32, const void* kcache, const void* vcache,
                                     const int* block_table, int bt_stride, const int* tok_seq,
                                     const int* tok_pos, void* out, int is_bf16, int N, int nq, int nkv,
                                     int d, int dv, int window, float scale, int layout, int v_layout,
                                     int chunk, float softcap, int sink, int v_in_k, const float* gate, int gS,
                                     long long g_split_stride, int g_width, int g_col0, cudaStream_t stream) {
    AttnOptions opt = {chunk, softcap, sink, v_in_k, gate, gS, g_split_stride, g_width, g_col0};
    if (gate && (gS < 1 || g_col0 < 0 || g_col0 + nq * dv > g_width)) return LUMEN_ERR_BAD_ARGUMENT;
    return attn_generic_launch(q, q_is_f32, kcache, vcache, block_table, bt_stride, tok_seq, tok_pos, out, is_bf16, N,
                               nq, nkv, d, dv, window, scale, layout, v_layout, opt, stream);
}
