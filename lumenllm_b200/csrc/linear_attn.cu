// Linear attention with a fixed decay a head: a recurrence over time with a matrix state per head,
//   S_t = decay_h S_(t-1) + k_t v_t^T  (S is d x dv),   o_t = S_t^T q_t,
// the token's own write seen by its own read. q, k (H heads of d) and v (H heads of dv) are columns
// of a projection that arrives as the S partial sums of a split product, [S, N, W] float32, added
// in rising order where a value is read; with `act` 1 each value goes through SiLU first. State,
// decay, sums and outputs are float32 whatever the run's type.
//
// A block takes one sequence, one head and a few columns of the state and walks the sequence's
// tokens of this step in order, the state in registers: a warp's lanes are PARTS parts x 32 / PARTS
// columns, part p holding rows p JPT .. p JPT + JPT of its column (d <= PARTS JPT; rows beyond d
// are zeros and stay zeros). The tokens' q, k and v come through shared memory in runs of LA_RUN
// tokens, staged by the whole block; the lanes of a part read the same q and k words, so a 16-byte
// shared load serves them in one go. An output is the sum of its column's parts, a few shuffles. Every number depends on its own sequence only and is made in the same order
// whatever the step's division into tokens, so prompts fed whole, in portions or token by token
// leave the same bits in the state.
//
// Two ways in. Steps of few tokens a sequence (decoding) read the projection's partial sums and apply
// the activation while they stage a run. Prompts first go through linear_attn_prep_kernel, which adds
// the partial sums and applies the activation ONCE for all blocks of a head (they share q and k) into
// a dense float32 buffer; the walk then fetches run r + 1 with 16-byte asynchronous copies into a
// second set of shared rows while it walks run r, and its token loop is unrolled so that a token's
// shuffles overlap the next token's state update.
#include "common.cuh"

#define LA_RUN 16
#define LA_GROUP 8
#define LA_THREADS 128

__device__ __forceinline__ float la_parts_sum(const float* p, int S, size_t stride) {
    float x = p[0];
    for (int s = 1; s < S; ++s) x += p[(size_t)s * stride];
    return x;
}
__device__ __forceinline__ float la_act(float x, int act) { return act ? x / (1.0f + expf(-x)) : x; }

// dense[n, c] = act(sum of the partial sums of u[n, c0 + c]) for the Wd columns of q, k and v.
__global__ void __launch_bounds__(256)
linear_attn_prep_kernel(const float* __restrict__ u, int S, size_t split_stride, int W, int q_col, int k_col, int v_col,
                        int Hd, int Hdv, int act, float* __restrict__ dense, long long total) {
    // No early trigger here: the walk that follows has fewer blocks than there are SMs and must find the
    // SMs empty, so that its blocks are spread one an SM; started under this kernel's blocks they are
    // packed several an SM wherever room is, and the walk takes twice as long (858 against 460 us for a
    // prompt of 2,048 tokens at 16 heads of 128 x 128).
    pdl_wait();
    const int Wd = 2 * Hd + Hdv;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const long long n = i / Wd;
        const int c = (int)(i - n * Wd);
        const int src = c < Hd ? q_col + c : (c < 2 * Hd ? k_col + c - Hd : v_col + c - 2 * Hd);
        dense[i] = la_act(la_parts_sum(u + n * W + src, S, split_stride), act);
    }
}

__device__ __forceinline__ void la_cp16(float* dst, const float* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}

// PRE: u is the dense buffer of linear_attn_prep_kernel (S = 1, no activation left to apply, q, k and v
// at columns that are multiples of 4, d and dv multiples of 4). PARTS lanes share a column (d <= PARTS *
// JPT), a warp holds CW = 32 / PARTS columns, a block 4 CW. In shared memory a token's q (and k) row is
// PARTS segments of JPT + 4 values: the 4 values of padding put the segments that a warp reads together
// on different banks (segments of 4 values need none: 32 lanes then read 512 bytes in a row).
template <int JPT, int PARTS, bool PRE>
__global__ void __launch_bounds__(LA_THREADS)
linear_attn_kernel(const float* __restrict__ u, int S, size_t split_stride, int W, int q_col, int k_col, int v_col,
                   int act, const float* __restrict__ decay, float* __restrict__ state, size_t slot_stride,
                   const int* __restrict__ cu_q, const int* __restrict__ seq_slot, float* __restrict__ out, int H, int d,
                   int dv) {
    constexpr int CW = 32 / PARTS, COLS = 4 * CW;   // columns a warp and a block
    constexpr int SEG = JPT + (JPT == 4 ? 0 : 4), DR = PARTS * SEG;  // a part's segment and a token's row of q (or k)
    constexpr int BUF = LA_RUN * (2 * DR + COLS);
    extern __shared__ __align__(16) float sm[];     // q [LA_RUN][DR], k [LA_RUN][DR], v [LA_RUN][COLS]; twice when PRE
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int part = lane / CW, e_local = lane % CW;
    const int e0 = blockIdx.x * COLS, h = blockIdx.y, b = blockIdx.z;
    const int e = e0 + warp * CW + e_local;
    const float a = decay[h];
    pdl_trigger();
    pdl_wait();
    const int t0 = cu_q[b], t1 = cu_q[b + 1];
    if (t1 <= t0) return;
    float* Sg = state + (size_t)seq_slot[b] * slot_stride + (size_t)h * d * dv;
    float st[JPT];
#pragma unroll
    for (int i = 0; i < JPT; ++i) {
        const int j = part * JPT + i;
        st[i] = (j < d && e < dv) ? Sg[(size_t)j * dv + e] : 0.0f;
    }
    // one token: the state moves on; what comes back is this part's share of the column's output
    auto token = [&](const float* qs, const float* ks, const float* vs, int t) -> float {
        const float v = vs[t * COLS];
        const float4* q4 = reinterpret_cast<const float4*>(qs + t * DR);
        const float4* k4 = reinterpret_cast<const float4*>(ks + t * DR);
        float o0 = 0.0f, o1 = 0.0f, o2 = 0.0f, o3 = 0.0f;
#pragma unroll
        for (int i = 0; i < JPT / 4; ++i) {
            const float4 q = q4[i], k = k4[i];
            st[4 * i] = fmaf(a, st[4 * i], k.x * v);
            st[4 * i + 1] = fmaf(a, st[4 * i + 1], k.y * v);
            st[4 * i + 2] = fmaf(a, st[4 * i + 2], k.z * v);
            st[4 * i + 3] = fmaf(a, st[4 * i + 3], k.w * v);
            o0 = fmaf(st[4 * i], q.x, o0);
            o1 = fmaf(st[4 * i + 1], q.y, o1);
            o2 = fmaf(st[4 * i + 2], q.z, o2);
            o3 = fmaf(st[4 * i + 3], q.w, o3);
        }
        return (o0 + o1) + (o2 + o3);
    };
    // One run of staged tokens, walked in order. A warp issues in order, so a token's chain of shuffles
    // (each waits for the one before) would hold up the next token's sums: LA_GROUP tokens' shares are
    // kept and summed over the parts together, their chains side by side. A full run is unrolled.
    auto walk = [&](const float* qs, const float* ks, const float* vs, int r0, int nt) {
        qs += part * SEG;
        ks += part * SEG;
        vs += warp * CW + e_local;
        float* orow = out + (size_t)r0 * H * dv + h * dv + e;
        const bool writes = part == 0 && e < dv;
        int t = 0;
        if (nt == LA_RUN) {
#pragma unroll
            for (int g0 = 0; g0 < LA_RUN; g0 += LA_GROUP) {
                float o[LA_GROUP];
#pragma unroll
                for (int g = 0; g < LA_GROUP; ++g) o[g] = token(qs, ks, vs, g0 + g);
#pragma unroll
                for (int x = CW; x < 32; x <<= 1)
#pragma unroll
                    for (int g = 0; g < LA_GROUP; ++g) o[g] += __shfl_xor_sync(0xffffffffu, o[g], x);
                if (writes)
#pragma unroll
                    for (int g = 0; g < LA_GROUP; ++g) orow[(size_t)(g0 + g) * H * dv] = o[g];
            }
            t = LA_RUN;
        }
        for (; t < nt; ++t) {
            float o = token(qs, ks, vs, t);
#pragma unroll
            for (int x = CW; x < 32; x <<= 1) o += __shfl_xor_sync(0xffffffffu, o, x);
            if (writes) orow[(size_t)t * H * dv] = o;
        }
    };
    if (PRE) {
        // rows beyond d, the padding and columns beyond dv are zeros in both sets and are never copied over
        for (int i = tid; i < 2 * BUF; i += LA_THREADS) sm[i] = 0.0f;
        __syncthreads();
        const int qc = d >> 2, pieces = 2 * qc + COLS / 4;       // 16-byte pieces a token: q, k, v
        auto fetch = [&](int r0, int nt, float* buf) {
            for (int i = tid; i < nt * pieces; i += LA_THREADS) {
                const int t = i / pieces, c = i - t * pieces;
                const float* row = u + (size_t)(r0 + t) * W;
                if (c < 2 * qc) {
                    const int j = 4 * (c < qc ? c : c - qc);          // JPT is a multiple of 4: a piece lies in one segment
                    la_cp16(buf + (c < qc ? 0 : LA_RUN * DR) + t * DR + (j / JPT) * SEG + j % JPT,
                            row + (c < qc ? q_col : k_col) + h * d + j);
                } else if (e0 + 4 * (c - 2 * qc) < dv) {
                    la_cp16(buf + 2 * LA_RUN * DR + t * COLS + 4 * (c - 2 * qc), row + v_col + h * dv + e0 + 4 * (c - 2 * qc));
                }
            }
            asm volatile("cp.async.commit_group;" ::: "memory");
        };
        fetch(t0, min(LA_RUN, t1 - t0), sm);
        int which = 0;
        for (int r0 = t0; r0 < t1; r0 += LA_RUN, which ^= 1) {
            const int nt = min(LA_RUN, t1 - r0);
            float* buf = sm + which * BUF;
            if (r0 + LA_RUN < t1) {
                fetch(r0 + LA_RUN, min(LA_RUN, t1 - r0 - LA_RUN), sm + (which ^ 1) * BUF);
                asm volatile("cp.async.wait_group 1;" ::: "memory");
            } else {
                asm volatile("cp.async.wait_group 0;" ::: "memory");
            }
            __syncthreads();
            walk(buf, buf + LA_RUN * DR, buf + 2 * LA_RUN * DR, r0, nt);
            __syncthreads();            // before the run after the next is copied over this one
        }
    } else {
        float* qs = sm;
        float* ks = sm + LA_RUN * DR;
        float* vs = sm + 2 * LA_RUN * DR;
        for (int r0 = t0; r0 < t1; r0 += LA_RUN) {
            const int nt = min(LA_RUN, t1 - r0);
            __syncthreads();            // the run before has been walked
            for (int i = tid; i < nt * PARTS * JPT; i += LA_THREADS) {
                const int t = i / (PARTS * JPT), j = i - t * (PARTS * JPT);
                float qv = 0.0f, kv = 0.0f;
                if (j < d) {
                    const float* row = u + (size_t)(r0 + t) * W + h * d + j;
                    qv = la_act(la_parts_sum(row + q_col, S, split_stride), act);
                    kv = la_act(la_parts_sum(row + k_col, S, split_stride), act);
                }
                qs[t * DR + (j / JPT) * SEG + j % JPT] = qv;
                ks[t * DR + (j / JPT) * SEG + j % JPT] = kv;
            }
            for (int i = tid; i < nt * COLS; i += LA_THREADS) {
                const int t = i / COLS, c = i - t * COLS;
                vs[i] = e0 + c < dv
                    ? la_act(la_parts_sum(u + (size_t)(r0 + t) * W + v_col + h * dv + e0 + c, S, split_stride), act) : 0.0f;
            }
            __syncthreads();
            walk(qs, ks, vs, r0, nt);
        }
    }
#pragma unroll
    for (int i = 0; i < JPT; ++i) {
        const int j = part * JPT + i;
        if (j < d && e < dv) Sg[(size_t)j * dv + e] = st[i];
    }
}

// Largest key size the kernel takes.
LUMEN_API int lumen_linear_attn_max_dim() { return 4 * 128; }

// 1 if a step of N tokens in n_seqs sequences takes the prompt path (it then needs a dense float32
// buffer of N (2 H d + H dv) values): at least LA_PRE_TOKENS tokens a sequence on average, head sizes
// that are multiples of 4.
#define LA_PRE_TOKENS 32
LUMEN_API int lumen_linear_attn_wants_dense(int N, int n_seqs, int d, int dv) {
    return (n_seqs > 0 && (long long)N >= (long long)LA_PRE_TOKENS * n_seqs && !(d & 3) && !(dv & 3)) ? 1 : 0;
}

// u: [S, N, W] partial sums; decay float32 [H]; state float32, sequence b's at state + seq_slot[b] *
// slot_stride as [H][d][dv], updated in place; cu_q int32 [B + 1]; out float32 [N, H dv]; dense: float32
// scratch of N (2 H d + H dv) values, 16-byte aligned, or null for the direct path.
LUMEN_API int lumen_linear_attn(const float* u, int n_split, long long split_stride, int W, int q_col, int k_col,
                                int v_col, int act, const float* decay, float* state, long long slot_stride,
                                const int* cu_q, const int* seq_slot, int n_seqs, float* out, int H, int d, int dv,
                                float* dense, int N, cudaStream_t stream) {
    if (n_seqs <= 0) return 0;
    if (n_split < 1 || H <= 0 || d <= 0 || dv <= 0 || q_col < 0 || k_col < 0 || v_col < 0 || q_col + H * d > W ||
        k_col + H * d > W || v_col + H * dv > W)
        return LUMEN_ERR_BAD_ARGUMENT;
    if (d > lumen_linear_attn_max_dim() || H > 65535 || n_seqs > 65535) return LUMEN_ERR_UNSUPPORTED;
    const bool pre = dense != nullptr;
    if (pre) {
        if ((d & 3) || (dv & 3) || ((uintptr_t)dense & 15) || N <= 0) return LUMEN_ERR_BAD_ARGUMENT;
        const long long total = (long long)N * (2 * H * d + H * dv);
        long long blocks = (total + 255) / 256;
        if (blocks > 148 * 16) blocks = 148 * 16;
        lumen_launch(linear_attn_prep_kernel, dim3((int)blocks), dim3(256), 0, stream, u, n_split, (size_t)split_stride, W,
                     q_col, k_col, v_col, H * d, H * dv, act, dense, total);
        LUMEN_LAUNCH_CHECK();
        u = dense;
        W = 2 * H * d + H * dv;
        q_col = 0, k_col = H * d, v_col = 2 * H * d, act = 0, n_split = 1, split_stride = 0;
    }
    // Steps of few tokens: 4 lanes a column, a sector of the state a part. Prompts: 8 lanes a column, so a
    // token's chain of sums is half as long and twice as many warps walk. (16 lanes a column, two warps a
    // scheduler: 424 us as with 8 for one prompt of 2,048 tokens at 16 heads of 128 x 128, but 613 against
    // 546 us at 32 heads and 1,108 against 834 us for four prompts: every warp reads the whole q and k rows
    // from shared memory, for half as many columns' worth of sums.)
#define LA_GO(JPT_, PARTS_, PRE_)                                                                                    \
    do {                                                                                                             \
        constexpr int cols = 4 * (32 / PARTS_);                                                                      \
        const size_t smem = (size_t)(PRE_ ? 2 : 1) * LA_RUN * (2 * PARTS_ * (JPT_ + (JPT_ == 4 ? 0 : 4)) + cols) * sizeof(float); \
        auto kern = linear_attn_kernel<JPT_, PARTS_, PRE_>;                                                          \
        if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);    \
        lumen_launch(kern, dim3((dv + cols - 1) / cols, H, n_seqs), dim3(LA_THREADS), smem, stream, u, n_split,      \
                     (size_t)split_stride, W, q_col, k_col, v_col, act, decay, state, (size_t)slot_stride, cu_q,     \
                     seq_slot, out, H, d, dv);                                                                       \
    } while (0)
    if (pre) {
        if (d <= 32) LA_GO(4, 8, true);
        else if (d <= 64) LA_GO(8, 8, true);
        else if (d <= 128) LA_GO(16, 8, true);
        else if (d <= 256) LA_GO(32, 8, true);
        else LA_GO(64, 8, true);
    } else {
        if (d <= 32) LA_GO(8, 4, false);
        else if (d <= 64) LA_GO(16, 4, false);
        else if (d <= 128) LA_GO(32, 4, false);
        else if (d <= 256) LA_GO(64, 4, false);
        else LA_GO(128, 4, false);
    }
#undef LA_GO
    LUMEN_LAUNCH_CHECK();
    return 0;
}
