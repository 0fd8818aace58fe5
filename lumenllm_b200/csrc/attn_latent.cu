// Causal flash attention over a latent cache: ONE row a token, W = R + r values wide, that is the key
// of every query head, and whose first dv values are the value of every head as well. Queries come
// already carried into that space ([N, H, W], bfloat16), so all H heads of a token share every
// cached row and a block's rows are (token, head) pairs: 64 consecutive rows of the query matrix
// [N H, W] that belong to one sequence. The same kernel serves prompts and single decoded tokens.
//
// Keys are walked 32 at a time (half a page; tiles start at multiples of 32 in absolute position,
// so what a row computes depends only on its own position, never on the batch or on how a prompt
// was cut). A tile's rows arrive by one bulk asynchronous copy each (cp.async.bulk + mbarrier) into
// a two-stage ring whose rows lie W + 8 values apart, which keeps ldmatrix free of bank conflicts
// for every W that is a multiple of 16. Sixteen warps: warp (g, c) owns the 16 rows of row group
// g = warp % 4 and, of the value columns, the slice c = warp / 4. Per tile
//   S      warp (g, c) multiplies its 16 rows with keys 8c .. 8c+8 of the tile over all W values
//          (mma.sync m16n8k16, bfloat16 in, float32 accumulate, two chains of products) and leaves
//          the 16 x 8 scores in shared memory as float32;
//   softmax every warp reads the 16 x 32 scores of its row group (the four warps of a group compute
//          the same maxima and sums, bit for bit), scale and mask, online softmax in float32 with
//          exp2 of log2(e)-scaled scores, P rounded to bfloat16 for the product, the sum taken before;
//   O      warp (g, c) adds P times the columns [c DVS, (c+1) DVS) of the same staged rows.
// A row sees key j if j <= p and (no window or p - j < window). Every wait is bounded; when one runs
// out the block raises the error flag and returns.
#include "common.cuh"
#include "mma_utils.cuh"

#define AL_THREADS 512
#define AL_ROWS 64
#define AL_KEYS 32
#define AL_PAD 8
#define AL_SS 40            // floats a row of the score buffer lies apart from the next

template <int DVS>
__global__ void __launch_bounds__(AL_THREADS)
attn_latent_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ cache,
                   const int* __restrict__ block_table, int bt_stride, const int* __restrict__ cu_q,
                   const int* __restrict__ seq_start, int B, float* __restrict__ out, float* __restrict__ part,
                   size_t rows_total, int H, int W, int dv, int window, float scale_log2, int* __restrict__ err) {
    pdl_wait();      // nothing of this kernel touches global memory before this
    pdl_trigger();
    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ uint64_t full[2];
    const int WP = W + AL_PAD;
    __nv_bfloat16* qs = reinterpret_cast<__nv_bfloat16*>(smem);                   // [64][WP]
    __nv_bfloat16* ks = qs + (size_t)AL_ROWS * WP;                                // [2][32][WP]
    float* ss = reinterpret_cast<float*>(ks + (size_t)2 * AL_KEYS * WP);          // [64][AL_SS]

    // which sequence, which tile of its rows
    int tile = blockIdx.x, b = 0, rows_seq = 0;
    for (; b < B; ++b) {
        rows_seq = (cu_q[b + 1] - cu_q[b]) * H;
        const int nt = (rows_seq + AL_ROWS - 1) / AL_ROWS;
        if (tile < nt) break;
        tile -= nt;
    }
    if (b >= B) return;
    const int row0 = tile * AL_ROWS;                            // first row of the tile within the sequence
    const int nrows = min(AL_ROWS, rows_seq - row0);
    const size_t grow0 = (size_t)cu_q[b] * H + row0;            // the same row in q / out
    const int start = seq_start[b];
    const int pos_first = start + row0 / H, pos_last = start + (row0 + nrows - 1) / H;
    int j_lo = 0;
    if (window > 0 && pos_first - window + 1 > 0) j_lo = pos_first - window + 1;
    const int kt_lo = j_lo / AL_KEYS, kt_hi = pos_last / AL_KEYS;
    const int* bt = block_table + (size_t)b * bt_stride;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const int rg = warp & 3, c = warp >> 2;

    if (tid == 0) {
        mbar_init(&full[0], 1);
        mbar_init(&full[1], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    const uint32_t row_bytes = (uint32_t)W * 2u;
    auto issue = [&](int stage, int kt) {          // warp 0, a lane a row
        const int page = bt[kt / (LUMEN_PAGE / AL_KEYS)];
        const __nv_bfloat16* src = cache + ((size_t)page * LUMEN_PAGE + (kt % (LUMEN_PAGE / AL_KEYS)) * AL_KEYS) * W;
        if (lane == 0) mbar_expect_tx(&full[stage], AL_KEYS * row_bytes);
        __syncwarp();
        bulk_load(ks + ((size_t)stage * AL_KEYS + lane) * WP, src + (size_t)lane * W, row_bytes, &full[stage]);
    };
    if (warp == 0 && kt_lo + (int)blockIdx.y <= kt_hi) issue(0, kt_lo + blockIdx.y);

    // the tile's query rows, 16 bytes at a time; rows past the sequence's last are zeros
    {
        const int chunks = W / 8;
        const uint4* src = reinterpret_cast<const uint4*>(q + grow0 * W);
        for (int i = tid; i < AL_ROWS * chunks; i += AL_THREADS) {
            const int r = i / chunks, ch = i - r * chunks;
            uint4 v = make_uint4(0u, 0u, 0u, 0u);
            if (r < nrows) v = src[(size_t)r * chunks + ch];
            *reinterpret_cast<uint4*>(qs + (size_t)r * WP + ch * 8) = v;
        }
    }
    __syncthreads();

    // this thread's two rows of the group and their positions (-1: no such row, nothing is seen)
    const int r0 = 16 * rg + g, r1 = r0 + 8;
    const bool active = 16 * rg < nrows;
    const int p0 = r0 < nrows ? start + (row0 + r0) / H : -1;
    const int p1 = r1 < nrows ? start + (row0 + r1) / H : -1;
    const int lo0 = window > 0 ? p0 - window + 1 : 0, lo1 = window > 0 ? p1 - window + 1 : 0;

    float o[DVS / 8][4];
#pragma unroll
    for (int i = 0; i < DVS / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.0f, l1 = 0.0f;
    bool failed = false;

    const uint32_t qs_a = smem_u32(qs) + (uint32_t)(((16 * rg + (lane & 7) + ((lane >> 3) & 1) * 8) * WP + (lane >> 4) * 8) * 2);
    const int ksteps = W / 16;

    const int n_split = gridDim.y, sp = blockIdx.y;     // block sp walks every n_split-th tile of keys
    for (int kt = kt_lo + sp, it = 0; kt <= kt_hi; kt += n_split, ++it) {
        const int stage = it & 1;
        if (warp == 0 && kt + n_split <= kt_hi) issue(stage ^ 1, kt + n_split);
        if (!mbar_wait(&full[stage], (it >> 1) & 1)) failed = true;
        const uint32_t kbase = smem_u32(ks + (size_t)stage * AL_KEYS * WP);

        if (active) {
            float a0[4] = {0.0f, 0.0f, 0.0f, 0.0f}, a1[4] = {0.0f, 0.0f, 0.0f, 0.0f};
            const uint32_t kb = kbase + (uint32_t)(((8 * c + (lane & 7)) * WP + (lane >> 3) * 8) * 2);
            int s2 = 0;
            for (; s2 + 1 < ksteps; s2 += 2) {
                uint32_t qa[4], qb[4], kr[4];
                ldsm_x4(kr, kb + s2 * 32);
                ldsm_x4(qa, qs_a + s2 * 32);
                ldsm_x4(qb, qs_a + s2 * 32 + 32);
                mma_bf16(a0, qa, kr[0], kr[1]);
                mma_bf16(a1, qb, kr[2], kr[3]);
            }
            if (s2 < ksteps) {      // an odd number of steps: the load's second half reads the padding and is not used
                uint32_t qa[4], kr[4];
                ldsm_x4(kr, kb + s2 * 32);
                ldsm_x4(qa, qs_a + s2 * 32);
                mma_bf16(a0, qa, kr[0], kr[1]);
            }
            *reinterpret_cast<float2*>(ss + r0 * AL_SS + 8 * c + 2 * t) = make_float2(a0[0] + a1[0], a0[1] + a1[1]);
            *reinterpret_cast<float2*>(ss + r1 * AL_SS + 8 * c + 2 * t) = make_float2(a0[2] + a1[2], a0[3] + a1[3]);
        }
        __syncthreads();
        if (active) {
            float s[4][4];
            const int jb = kt * AL_KEYS;
            float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
            for (int nt = 0; nt < 4; ++nt) {
                const float2 u0 = *reinterpret_cast<const float2*>(ss + r0 * AL_SS + 8 * nt + 2 * t);
                const float2 u1 = *reinterpret_cast<const float2*>(ss + r1 * AL_SS + 8 * nt + 2 * t);
                const int j = jb + 8 * nt + 2 * t;
                s[nt][0] = (j <= p0 && j >= lo0) ? u0.x * scale_log2 : -INFINITY;
                s[nt][1] = (j + 1 <= p0 && j + 1 >= lo0) ? u0.y * scale_log2 : -INFINITY;
                s[nt][2] = (j <= p1 && j >= lo1) ? u1.x * scale_log2 : -INFINITY;
                s[nt][3] = (j + 1 <= p1 && j + 1 >= lo1) ? u1.y * scale_log2 : -INFINITY;
                mx0 = fmaxf(mx0, fmaxf(s[nt][0], s[nt][1]));
                mx1 = fmaxf(mx1, fmaxf(s[nt][2], s[nt][3]));
            }
            mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
            mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
            mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
            mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
            const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
            const float ms0 = (mn0 == -INFINITY) ? 0.0f : mn0, ms1 = (mn1 == -INFINITY) ? 0.0f : mn1;
            const float c0 = (m0 == -INFINITY) ? 0.0f : exp2f(m0 - ms0);
            const float c1 = (m1 == -INFINITY) ? 0.0f : exp2f(m1 - ms1);
            float rs0 = 0.0f, rs1 = 0.0f;
#pragma unroll
            for (int nt = 0; nt < 4; ++nt) {
                s[nt][0] = exp2f(s[nt][0] - ms0);
                s[nt][1] = exp2f(s[nt][1] - ms0);
                s[nt][2] = exp2f(s[nt][2] - ms1);
                s[nt][3] = exp2f(s[nt][3] - ms1);
                rs0 += s[nt][0] + s[nt][1];
                rs1 += s[nt][2] + s[nt][3];
            }
            rs0 += __shfl_xor_sync(0xffffffffu, rs0, 1);
            rs0 += __shfl_xor_sync(0xffffffffu, rs0, 2);
            rs1 += __shfl_xor_sync(0xffffffffu, rs1, 1);
            rs1 += __shfl_xor_sync(0xffffffffu, rs1, 2);
            l0 = l0 * c0 + rs0;
            l1 = l1 * c1 + rs1;
            m0 = mn0;
            m1 = mn1;
            uint32_t pa[2][4];
#pragma unroll
            for (int kk = 0; kk < 2; ++kk) {
                pa[kk][0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
                pa[kk][1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
                pa[kk][2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
                pa[kk][3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
            }
            const int mi = lane >> 3;
            const uint32_t vb = kbase + (uint32_t)((((mi & 1) * 8 + (lane & 7)) * WP + c * DVS + (mi >> 1) * 8) * 2);
#pragma unroll
            for (int np = 0; np < DVS / 16; ++np) {
                if (c * DVS + 16 * np < dv) {
                    o[2 * np][0] *= c0; o[2 * np][1] *= c0; o[2 * np][2] *= c1; o[2 * np][3] *= c1;
                    o[2 * np + 1][0] *= c0; o[2 * np + 1][1] *= c0; o[2 * np + 1][2] *= c1; o[2 * np + 1][3] *= c1;
#pragma unroll
                    for (int kk = 0; kk < 2; ++kk) {
                        uint32_t r[4];
                        ldsm_x4_t(r, vb + (uint32_t)((16 * kk * WP + 16 * np) * 2));
                        mma_bf16(o[2 * np], pa[kk], r[0], r[1]);
                        mma_bf16(o[2 * np + 1], pa[kk], r[2], r[3]);
                    }
                }
            }
        }
        // every warp is done with this stage and with the scores before either is written again
        if (__syncthreads_or(failed)) {
            if (tid == 0) atomicExch(err, 1);
            return;
        }
    }

    if (!active) return;
    if (n_split > 1) {
        // this block's share, not normed: [o (dv) | running maximum (log2 units), running sum] a row
        float* p0r = part + ((size_t)sp * rows_total + grow0 + r0) * (dv + 2);
        float* p1r = part + ((size_t)sp * rows_total + grow0 + r1) * (dv + 2);
#pragma unroll
        for (int nt = 0; nt < DVS / 8; ++nt) {
            const int col = c * DVS + 8 * nt + 2 * t;
            if (col < dv) {
                if (r0 < nrows) *reinterpret_cast<float2*>(p0r + col) = make_float2(o[nt][0], o[nt][1]);
                if (r1 < nrows) *reinterpret_cast<float2*>(p1r + col) = make_float2(o[nt][2], o[nt][3]);
            }
        }
        if (c == 0 && t == 0) {
            if (r0 < nrows) *reinterpret_cast<float2*>(p0r + dv) = make_float2(m0, l0);
            if (r1 < nrows) *reinterpret_cast<float2*>(p1r + dv) = make_float2(m1, l1);
        }
        return;
    }
    const float inv0 = (l0 > 0.0f) ? 1.0f / l0 : 0.0f, inv1 = (l1 > 0.0f) ? 1.0f / l1 : 0.0f;
    float* o0 = out + (grow0 + r0) * dv;
    float* o1 = out + (grow0 + r1) * dv;
#pragma unroll
    for (int nt = 0; nt < DVS / 8; ++nt) {
        const int col = c * DVS + 8 * nt + 2 * t;
        if (col < dv) {
            if (r0 < nrows) *reinterpret_cast<float2*>(o0 + col) = make_float2(o[nt][0] * inv0, o[nt][1] * inv0);
            if (r1 < nrows) *reinterpret_cast<float2*>(o1 + col) = make_float2(o[nt][2] * inv1, o[nt][3] * inv1);
        }
    }
}

// The shares of a row's n_split blocks become the row: out = sum_s 2^(m_s - M) o_s / sum_s 2^(m_s - M) l_s,
// always in the order of s. A block a row.
#define AL_MAX_SPLIT 16
__global__ void __launch_bounds__(128)
attn_latent_merge_kernel(const float* __restrict__ part, float* __restrict__ out, size_t rows_total, int dv, int n_split) {
    pdl_wait();
    pdl_trigger();
    const size_t row = blockIdx.x;
    float w[AL_MAX_SPLIT];
    float M = -INFINITY, L = 0.0f;
    for (int s = 0; s < n_split; ++s) M = fmaxf(M, part[((size_t)s * rows_total + row) * (dv + 2) + dv]);
    for (int s = 0; s < n_split; ++s) {
        const float* p = part + ((size_t)s * rows_total + row) * (dv + 2) + dv;
        w[s] = (p[0] == -INFINITY) ? 0.0f : exp2f(p[0] - M);
        L += w[s] * p[1];
    }
    const float inv = L > 0.0f ? 1.0f / L : 0.0f;
    for (int e = threadIdx.x; e < dv; e += 128) {
        float acc = 0.0f;
        for (int s = 0; s < n_split; ++s)
            if (w[s] != 0.0f) acc = fmaf(w[s], part[((size_t)s * rows_total + row) * (dv + 2) + e], acc);
        out[row * dv + e] = acc * inv;
    }
}

// Shared memory the kernel asks for with rows of W values.
static inline size_t attn_latent_smem(int W) {
    return (size_t)(AL_ROWS + 2 * AL_KEYS) * (W + AL_PAD) * 2 + (size_t)AL_ROWS * AL_SS * sizeof(float);
}

// 1 if lumen_attn_latent takes rows of W values with dv of them the value.
LUMEN_API int lumen_attn_latent_takes(int W, int dv) {
    return (W > 0 && W % 16 == 0 && dv > 0 && dv % 8 == 0 && dv <= W && dv <= 512 &&
            attn_latent_smem(W) <= 227 * 1024) ? 1 : 0;
}

// q bfloat16 [N, H, W]; cache bfloat16 [pages, 1, PAGE, W] (plain tiles); out float32 [N, H, dv];
// cu_q int32 [B+1]; seq_start int32 [B] (cached length of each sequence before this step);
// n_tiles >= the sum over sequences of ceil(q_len H / 64) (blocks left over return at once).
// n_split > 1 (steps of few rows, as decode steps are): a row's keys are shared out among n_split
// blocks, tile by tile in turn, and merged by a second kernel; part then holds
// n_split * N * H * (dv + 2) floats of scratch. How a row's keys are shared out depends on n_split and
// the row's own position alone.
LUMEN_API int lumen_attn_latent(const void* q, const void* cache, const int* block_table, int bt_stride,
                                const int* cu_q, const int* seq_start, int B, int n_tiles, void* out, void* part,
                                int n_split, int N, int H, int W, int dv, int window, float scale, int* err,
                                cudaStream_t stream) {
    if (B <= 0 || n_tiles <= 0 || N <= 0) return 0;
    if (H <= 0 || window < 0 || !lumen_attn_latent_takes(W, dv)) return LUMEN_ERR_UNSUPPORTED;
    if (n_split < 1 || n_split > AL_MAX_SPLIT || (n_split > 1 && !part)) return LUMEN_ERR_BAD_ARGUMENT;
    const size_t rows_total = (size_t)N * H;
    const float scale_log2 = scale * 1.4426950408889634f;
    const size_t smem = attn_latent_smem(W);
    const __nv_bfloat16* qp = (const __nv_bfloat16*)q;
    const __nv_bfloat16* cp = (const __nv_bfloat16*)cache;
#define AL_LAUNCH(S)                                                                                              \
    do {                                                                                                          \
        auto k = attn_latent_kernel<S>;                                                                           \
        cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);          \
        if (e != cudaSuccess) return (int)e;                                                                      \
        lumen_launch(k, dim3(n_tiles, n_split), dim3(AL_THREADS), smem, stream, qp, cp, block_table, bt_stride,   \
                     cu_q, seq_start, B, (float*)out, (float*)part, rows_total, H, W, dv, window, scale_log2,     \
                     err);                                                                                        \
    } while (0)
    if (dv <= 128) AL_LAUNCH(32);
    else if (dv <= 256) AL_LAUNCH(64);
    else AL_LAUNCH(128);
#undef AL_LAUNCH
    LUMEN_LAUNCH_CHECK();
    if (n_split > 1) {
        if (rows_total > 0x7fffffffu) return LUMEN_ERR_UNSUPPORTED;
        lumen_launch(attn_latent_merge_kernel, dim3((unsigned)rows_total), dim3(128), 0, stream, (const float*)part,
                     (float*)out, rows_total, dv, n_split);
        LUMEN_LAUNCH_CHECK();
    }
    return 0;
}
