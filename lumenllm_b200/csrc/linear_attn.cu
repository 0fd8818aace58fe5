// Linear attention with a fixed decay a head: a recurrence over time with a matrix state per head,
//   S_t = decay_h S_(t-1) + k_t v_t^T  (S is d x dv),   o_t = S_t^T q_t,
// the token's own write seen by its own read. q, k (H heads of d) and v (H heads of dv) are columns
// of a projection that arrives as the S partial sums of a split product, [S, N, W] float32, added
// in rising order where a value is read; with `act` 1 each value goes through SiLU first. State,
// decay, sums and outputs are float32 whatever the run's type.
//
// A block takes one sequence, one head and LA_COLS columns of the state and walks the sequence's
// tokens of this step in order, the state in registers: a warp holds 8 columns, its lanes are
// 4 parts x 8 columns, part p holding rows p JPT .. p JPT + JPT of its column (d <= 4 JPT; rows
// beyond d are zeros and stay zeros). The tokens' q, k and v come through shared memory in runs of
// LA_RUN tokens, staged by the whole block; the 8 lanes of a quarter warp read the same q and k
// words, so a 16-byte shared load serves them in one go. An output is the sum of its column's 4
// parts, two shuffles. Every number depends on its own sequence only and is made in the same order
// whatever the step's division into tokens, so prompts fed whole, in portions or token by token
// leave the same bits in the state.
#include "common.cuh"

#define LA_COLS 32
#define LA_RUN 16
#define LA_THREADS 128

__device__ __forceinline__ float la_parts_sum(const float* p, int S, size_t stride) {
    float x = p[0];
    for (int s = 1; s < S; ++s) x += p[(size_t)s * stride];
    return x;
}
__device__ __forceinline__ float la_act(float x, int act) { return act ? x / (1.0f + expf(-x)) : x; }

template <int JPT>
__global__ void __launch_bounds__(LA_THREADS)
linear_attn_kernel(const float* __restrict__ u, int S, size_t split_stride, int W, int q_col, int k_col, int v_col,
                   int act, const float* __restrict__ decay, float* __restrict__ state, size_t slot_stride,
                   const int* __restrict__ cu_q, const int* __restrict__ seq_slot, float* __restrict__ out, int H, int d,
                   int dv) {
    constexpr int DR = 4 * JPT;                     // padded rows of q and k a token
    extern __shared__ __align__(16) float sm[];     // q [LA_RUN][DR], k [LA_RUN][DR], v [LA_RUN][LA_COLS]
    float* qs = sm;
    float* ks = sm + LA_RUN * DR;
    float* vs = sm + 2 * LA_RUN * DR;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int part = lane >> 3, e_local = lane & 7;
    const int e0 = blockIdx.x * LA_COLS, h = blockIdx.y, b = blockIdx.z;
    const int e = e0 + warp * 8 + e_local;
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
    for (int r0 = t0; r0 < t1; r0 += LA_RUN) {
        const int nt = min(LA_RUN, t1 - r0);
        __syncthreads();            // the run before has been walked
        for (int i = tid; i < nt * DR; i += LA_THREADS) {
            const int t = i / DR, j = i - t * DR;
            float qv = 0.0f, kv = 0.0f;
            if (j < d) {
                const float* row = u + (size_t)(r0 + t) * W + h * d + j;
                qv = la_act(la_parts_sum(row + q_col, S, split_stride), act);
                kv = la_act(la_parts_sum(row + k_col, S, split_stride), act);
            }
            qs[i] = qv;
            ks[i] = kv;
        }
        for (int i = tid; i < nt * LA_COLS; i += LA_THREADS) {
            const int t = i / LA_COLS, c = i - t * LA_COLS;
            vs[i] = e0 + c < dv
                ? la_act(la_parts_sum(u + (size_t)(r0 + t) * W + v_col + h * dv + e0 + c, S, split_stride), act) : 0.0f;
        }
        __syncthreads();
        for (int t = 0; t < nt; ++t) {
            const float v = vs[t * LA_COLS + warp * 8 + e_local];
            const float4* q4 = reinterpret_cast<const float4*>(qs + t * DR + part * JPT);
            const float4* k4 = reinterpret_cast<const float4*>(ks + t * DR + part * JPT);
            float o0 = 0.0f, o1 = 0.0f;
#pragma unroll
            for (int i = 0; i < JPT / 4; ++i) {
                const float4 q = q4[i], k = k4[i];
                st[4 * i] = fmaf(a, st[4 * i], k.x * v);
                st[4 * i + 1] = fmaf(a, st[4 * i + 1], k.y * v);
                st[4 * i + 2] = fmaf(a, st[4 * i + 2], k.z * v);
                st[4 * i + 3] = fmaf(a, st[4 * i + 3], k.w * v);
                o0 = fmaf(st[4 * i], q.x, o0);
                o1 = fmaf(st[4 * i + 1], q.y, o1);
                o0 = fmaf(st[4 * i + 2], q.z, o0);
                o1 = fmaf(st[4 * i + 3], q.w, o1);
            }
            float o = o0 + o1;
            o += __shfl_xor_sync(0xffffffffu, o, 8);
            o += __shfl_xor_sync(0xffffffffu, o, 16);
            if (part == 0 && e < dv) out[(size_t)(r0 + t) * H * dv + h * dv + e] = o;
        }
    }
#pragma unroll
    for (int i = 0; i < JPT; ++i) {
        const int j = part * JPT + i;
        if (j < d && e < dv) Sg[(size_t)j * dv + e] = st[i];
    }
}

// Largest key size the kernel takes.
LUMEN_API int lumen_linear_attn_max_dim() { return 4 * 64; }

// u: [S, N, W] partial sums; decay float32 [H]; state float32, sequence b's at state + seq_slot[b] *
// slot_stride as [H][d][dv], updated in place; cu_q int32 [B + 1]; out float32 [N, H dv].
LUMEN_API int lumen_linear_attn(const float* u, int n_split, long long split_stride, int W, int q_col, int k_col,
                                int v_col, int act, const float* decay, float* state, long long slot_stride,
                                const int* cu_q, const int* seq_slot, int n_seqs, float* out, int H, int d, int dv,
                                cudaStream_t stream) {
    if (n_seqs <= 0) return 0;
    if (n_split < 1 || H <= 0 || d <= 0 || dv <= 0 || q_col < 0 || k_col < 0 || v_col < 0 || q_col + H * d > W ||
        k_col + H * d > W || v_col + H * dv > W)
        return LUMEN_ERR_BAD_ARGUMENT;
    if (d > lumen_linear_attn_max_dim() || H > 65535 || n_seqs > 65535) return LUMEN_ERR_UNSUPPORTED;
    dim3 grid((dv + LA_COLS - 1) / LA_COLS, H, n_seqs);
#define LA_GO(JPT_)                                                                                                  \
    do {                                                                                                             \
        const size_t smem = (size_t)LA_RUN * (2 * 4 * JPT_ + LA_COLS) * sizeof(float);                               \
        auto kern = linear_attn_kernel<JPT_>;                                                                        \
        if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);    \
        lumen_launch(kern, grid, dim3(LA_THREADS), smem, stream, u, n_split, (size_t)split_stride, W, q_col, k_col,  \
                     v_col, act, decay, state, (size_t)slot_stride, cu_q, seq_slot, out, H, d, dv);                  \
    } while (0)
    if (d <= 32) LA_GO(8);
    else if (d <= 64) LA_GO(16);
    else if (d <= 128) LA_GO(32);
    else LA_GO(64);
#undef LA_GO
    LUMEN_LAUNCH_CHECK();
    return 0;
}
