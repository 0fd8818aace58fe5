// A feed-forward made of many small experts of which each token uses a few.
//   1. route: softmax over the router's logits (float32) or, mode 1, a sigmoid of each logit by
//      itself; choice by score + a correction, the chosen experts' scores (without the correction)
//      times a scale as weights.
//   2. group: the step's (token, choice) entries put in order of their expert, and the list of
//      row tiles (expert, first entry, number of entries) that the products walk. Everything
//      stays on the device: the products are launched with as many blocks as any routing can
//      need, and the blocks beyond the list leave.
//   3. two grouped products: gate and up with SiLU(gate) * up behind them, then down with the
//      entry's weight, written to out[choice][token][:] so that the consumer adds a token's
//      choices in rising order, like the partial sums of a split product. The entry's weight may
//      multiply the expert's INPUT instead: the gated product then multiplies its two sums by it
//      before the activation (a product is linear in its input), and the down product gets no
//      weights. Activation 1 is the clamped unit g sigmoid(alpha g) (v + 1) with g = min(gate, limit),
//      v = clamp(up, -limit, limit).
//   4. identity experts (indices from n_experts on): out[choice][token][:] = weight * input,
//      written by the routing kernel, which has the token's row at hand.
// Every output element is one dot product summed over k in rising order by one thread, so it
// depends on its own row and the expert's weights only, never on the batch or on the order in
// which the entries of an expert were listed.
#include "common.cuh"
#include "mma_utils.cuh"

#define MOE_MAX_LANE_VALS 16      // router outputs a lane holds: up to 512 experts
#define MOE_MAX_EXPERTS 1024
#define MOE_TM 32                 // entries a row tile (32-bit products)
#define MOE_TM_MMA 64             // entries a row tile (tensor-core products, many entries an expert)
#define MOE_TM_MMA_FEW 16         // entries a row tile (tensor-core products, few entries an expert)
#define MOE_TN 64                 // output columns a block
#define MOE_TK 32

// ---------------------------------------------------------------- route
// A warp a token. logits float32 [N, Et]; corr float32 [Et] or null; idx int32 [N, top];
// wt float32 [N, top]. Equal choice scores go to the lower index.
__device__ __forceinline__ void route_row(const float* __restrict__ lg, const float* __restrict__ corr, int Et,
                                          int top, float scale, int* __restrict__ idx, float* __restrict__ wt, int lane,
                                          int mode) {
    float s[MOE_MAX_LANE_VALS], c[MOE_MAX_LANE_VALS];
    float m = -INFINITY;
    if (mode == 1) {            // every score by itself: 1 / (1 + exp(-logit))
#pragma unroll
        for (int r = 0; r < MOE_MAX_LANE_VALS; ++r) {
            const int e = lane + 32 * r;
            s[r] = e < Et ? 1.0f / (1.0f + expf(-lg[e])) : 0.0f;
            c[r] = e < Et ? s[r] + (corr ? corr[e] : 0.0f) : -INFINITY;
        }
    } else {
#pragma unroll
    for (int r = 0; r < MOE_MAX_LANE_VALS; ++r) {
        const int e = lane + 32 * r;
        s[r] = e < Et ? lg[e] : -INFINITY;
        m = fmaxf(m, s[r]);
    }
    m = warp_max(m);
    float sum = 0.0f;
#pragma unroll
    for (int r = 0; r < MOE_MAX_LANE_VALS; ++r) {
        const int e = lane + 32 * r;
        s[r] = e < Et ? expf(s[r] - m) : 0.0f;
        sum += s[r];
    }
    sum = warp_sum(sum);
    const float inv = 1.0f / sum;
#pragma unroll
    for (int r = 0; r < MOE_MAX_LANE_VALS; ++r) {
        const int e = lane + 32 * r;
        s[r] *= inv;
        c[r] = e < Et ? s[r] + (corr ? corr[e] : 0.0f) : -INFINITY;
    }
    }
    for (int k = 0; k < top; ++k) {
        float best = -INFINITY, best_s = 0.0f;
        int best_e = 0x7fffffff;
#pragma unroll
        for (int r = 0; r < MOE_MAX_LANE_VALS; ++r) {
            const int e = lane + 32 * r;
            if (e < Et && (c[r] > best || (c[r] == best && e < best_e))) { best = c[r]; best_e = e; best_s = s[r]; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
            const float os = __shfl_xor_sync(0xffffffffu, best_s, o);
            if (ob > best || (ob == best && oe < best_e)) { best = ob; best_e = oe; best_s = os; }
        }
#pragma unroll
        for (int r = 0; r < MOE_MAX_LANE_VALS; ++r)
            if (lane + 32 * r == best_e) c[r] = -INFINITY;        // taken
        if (lane == 0) {
            idx[k] = best_e;
            wt[k] = best_s * scale;
        }
    }
}

__global__ void __launch_bounds__(128)
moe_route_kernel(const float* __restrict__ logits, const float* __restrict__ corr, int Et, int top, float scale,
                 int* __restrict__ idx, float* __restrict__ wt, int N, int mode) {
    pdl_trigger();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (t >= N) return;
    route_row(logits + (size_t)t * Et, corr, Et, top, scale, idx + (size_t)t * top, wt + (size_t)t * top, lane, mode);
}

// The router's product and the choice in one kernel, a block a token: the token's row goes to
// shared memory as float32, every warp takes router rows in turn (W float32 [Et, K]; lanes
// strided over k, then a butterfly, so a logit's sum has one order whatever the batch), and the
// first warp routes. With ident_out the identity experts' share of the update is written here too.
template <typename TA>
__global__ void __launch_bounds__(1024)
moe_route_x_kernel(const TA* __restrict__ x, const float* __restrict__ W, int K, const float* __restrict__ corr, int Et,
                   int top, float scale, int* __restrict__ idx, float* __restrict__ wt, float* __restrict__ ident_out,
                   int E, int n_tokens, int mode) {
    extern __shared__ __align__(16) float rs[];      // K floats, then Et logits
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
    float* lg = rs + K;
    for (int i = threadIdx.x; i < K; i += blockDim.x) rs[i] = to_f32(x[(size_t)t * K + i]);
    __syncthreads();
    for (int e = warp; e < Et; e += nwarp) {
        const float* we = W + (size_t)e * K;
        float acc = 0.0f;
        if ((K & 3) == 0) {                       // four values a lane a turn, all loads of a row in flight
            float a1 = 0.0f, a2 = 0.0f, a3 = 0.0f;
#pragma unroll 8
            for (int i = lane * 4; i < K; i += 128) {
                const float4 wv = *reinterpret_cast<const float4*>(we + i);
                const float4 xv = *reinterpret_cast<const float4*>(rs + i);
                acc = fmaf(xv.x, wv.x, acc);
                a1 = fmaf(xv.y, wv.y, a1);
                a2 = fmaf(xv.z, wv.z, a2);
                a3 = fmaf(xv.w, wv.w, a3);
            }
            acc = (acc + a1) + (a2 + a3);
        } else {
            for (int i = lane; i < K; i += 32) acc = fmaf(rs[i], we[i], acc);
        }
        acc = warp_sum(acc);
        if (lane == 0) lg[e] = acc;
    }
    __syncthreads();
    if (warp == 0) route_row(lg, corr, Et, top, scale, idx + (size_t)t * top, wt + (size_t)t * top, lane, mode);
    if (!ident_out) return;
    // choices that fell on identity experts (indices from E on): the token's own row times the
    // weight, at the choice's place in the update's stack [top, tokens, K]
    __syncthreads();
    for (int k = 0; k < top; ++k) {
        if (idx[(size_t)t * top + k] < E) continue;
        const float w = wt[(size_t)t * top + k];
        float* o = ident_out + ((size_t)k * n_tokens + t) * K;
        for (int i = threadIdx.x; i < K; i += blockDim.x) o[i] = w * rs[i];
    }
}

LUMEN_API int lumen_moe_route_x(const void* x, int x_is_bf16, const float* W, int K, const float* corr, int Et, int top,
                                float scale, int* idx, float* wt, float* ident_out, int E, int N, int mode,
                                cudaStream_t stream) {
    if (N <= 0) return 0;
    if (Et <= 0 || top <= 0 || top > Et || K <= 0) return LUMEN_ERR_BAD_ARGUMENT;
    const size_t smem = (size_t)(K + Et) * sizeof(float);
    if (Et > 32 * MOE_MAX_LANE_VALS || smem > 200 * 1024) return LUMEN_ERR_UNSUPPORTED;
    // few tokens (decode steps): a warp a router row, all rows at once; many: 8 warps a token
    int threads = 256;
    if (N < 2 * 148) threads = Et >= 32 ? 1024 : (Et < 4 ? 128 : 32 * Et);
    if (x_is_bf16) {
        auto k = moe_route_x_kernel<__nv_bfloat16>;
        if (smem > 48 * 1024) cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        lumen_launch(k, dim3(N), dim3(threads), smem, stream, (const __nv_bfloat16*)x, W, K, corr, Et, top, scale, idx, wt,
                     ident_out, E, N, mode);
    } else {
        auto k = moe_route_x_kernel<float>;
        if (smem > 48 * 1024) cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        lumen_launch(k, dim3(N), dim3(threads), smem, stream, (const float*)x, W, K, corr, Et, top, scale, idx, wt, ident_out,
                     E, N, mode);
    }
    LUMEN_LAUNCH_CHECK();
    return 0;
}

LUMEN_API int lumen_moe_route(const float* logits, const float* corr, int Et, int top, float scale, int* idx,
                              float* wt, int N, int mode, cudaStream_t stream) {
    if (N <= 0) return 0;
    if (Et <= 0 || top <= 0 || top > Et) return LUMEN_ERR_BAD_ARGUMENT;
    if (Et > 32 * MOE_MAX_LANE_VALS) return LUMEN_ERR_UNSUPPORTED;
    lumen_launch(moe_route_kernel, dim3((N + 3) / 4), dim3(128), 0, stream, logits, corr, Et, top, scale, idx, wt, N, mode);
    LUMEN_LAUNCH_CHECK();
    return 0;
}

// ---------------------------------------------------------------- group
// One block. entries = N * top; sorted int32 [entries] receives the entries (token * top +
// choice) of expert 0, then of expert 1, ...; entries of identity experts (idx >= E) are left
// out. tiles int32 [max_tiles, 3] = (expert, first place in sorted, count <= tile_rows);
// n_tiles int32 [1].
__global__ void __launch_bounds__(1024)
moe_group_kernel(const int* __restrict__ idx, int entries, int E, int tile_rows, int* __restrict__ sorted,
                 int* __restrict__ tiles, int* __restrict__ n_tiles) {
    __shared__ int count[MOE_MAX_EXPERTS], start[MOE_MAX_EXPERTS];
    pdl_trigger();
    pdl_wait();
    for (int e = threadIdx.x; e < E; e += blockDim.x) count[e] = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < entries; i += blockDim.x) {
        const int e = idx[i];
        if (e >= 0 && e < E) atomicAdd(&count[e], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int at = 0, nt = 0;
        for (int e = 0; e < E; ++e) {
            const int c = count[e];
            start[e] = at;
            for (int o = 0; o < c; o += tile_rows) {
                tiles[3 * nt] = e;
                tiles[3 * nt + 1] = at + o;
                tiles[3 * nt + 2] = min(tile_rows, c - o);
                ++nt;
            }
            at += c;
            count[e] = 0;             // from here on: entries of e placed so far
        }
        *n_tiles = nt;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < entries; i += blockDim.x) {
        const int e = idx[i];
        if (e >= 0 && e < E) sorted[start[e] + atomicAdd(&count[e], 1)] = i;
    }
}

// Entries a row tile: of the tensor-core products (bfloat16 operands) and of the 32-bit ones.
// tensor_cores: 0 the 32-bit products, 1 the tensor-core products' tall tiles, 2 their short ones.
LUMEN_API int lumen_moe_tile_rows(int tensor_cores) {
    return tensor_cores == 2 ? MOE_TM_MMA_FEW : tensor_cores ? MOE_TM_MMA : MOE_TM;
}

LUMEN_API int lumen_moe_group(const int* idx, int entries, int E, int tile_rows, int* sorted, int* tiles,
                              int* n_tiles, cudaStream_t stream) {
    if (entries <= 0) return 0;
    if (E <= 0 || E > MOE_MAX_EXPERTS) return LUMEN_ERR_UNSUPPORTED;
    if (tile_rows != MOE_TM && tile_rows != MOE_TM_MMA && tile_rows != MOE_TM_MMA_FEW) return LUMEN_ERR_BAD_ARGUMENT;
    lumen_launch(moe_group_kernel, dim3(1), dim3(1024), 0, stream, idx, entries, E, tile_rows, sorted, tiles, n_tiles);
    LUMEN_LAUNCH_CHECK();
    return 0;
}

// ---------------------------------------------------------------- grouped products
// Block (tile, column block): the tile's entries x MOE_TN output columns of the tile's expert.
// GATED: the rows of the activations are tokens (entry / top); W is [E, 2 F, K], gate rows
//   first; out[entry, f] = act(w gate, w up) in the activations' type, w the entry's weight (1
//   when wt is null), act = silu(gate) * up or the clamped unit (MoeAct).
// else:  the rows of the activations are entries; W is [E, Nout, K]; out is float32
//   [top, tokens, Nout] and receives weight[entry] * product at [entry % top][entry / top].
// 256 threads; a thread holds 2 rows x 4 columns (of gate and of up when GATED).
struct MoeAct {
    int kind;            // 0: silu(g) * u; 1: min(g, limit) sigmoid(alpha min(g, limit)) (clamp(u, +-limit) + 1)
    float limit, alpha;
    __device__ __forceinline__ float of(float g, float u) const {
        if (kind == 1) {
            g = fminf(g, limit);
            u = fminf(fmaxf(u, -limit), limit);
            return g / (1.0f + expf(-alpha * g)) * (u + 1.0f);
        }
        return g / (1.0f + expf(-g)) * u;
    }
};
template <typename TA, typename TW, bool GATED>
__global__ void __launch_bounds__(256)
moe_product_kernel(const TA* __restrict__ A, const TW* __restrict__ W, const int* __restrict__ sorted,
                   const int* __restrict__ tiles, const int* __restrict__ n_tiles, const float* __restrict__ wt,
                   void* __restrict__ out, int K, int Nout, int top, int n_tokens, MoeAct act) {
    __shared__ float As[MOE_TK][MOE_TM + 1];
    __shared__ float Ws[GATED ? 2 : 1][MOE_TK][MOE_TN + 1];
    __shared__ int rows[MOE_TM];
    pdl_trigger();
    pdl_wait();
    const int tile = blockIdx.x;
    if (tile >= *n_tiles) return;
    const int e = tiles[3 * tile], first = tiles[3 * tile + 1], cnt = tiles[3 * tile + 2];
    const int n0 = blockIdx.y * MOE_TN;
    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    if (tid < MOE_TM) rows[tid] = tid < cnt ? sorted[first + tid] : -1;
    __syncthreads();
    const TW* We = W + (size_t)e * (GATED ? 2 : 1) * Nout * K;
    float acc[GATED ? 2 : 1][2][4];
#pragma unroll
    for (int m = 0; m < (GATED ? 2 : 1); ++m)
#pragma unroll
        for (int i = 0; i < 2; ++i)
#pragma unroll
            for (int jn = 0; jn < 4; ++jn) acc[m][i][jn] = 0.0f;
    for (int k0 = 0; k0 < K; k0 += MOE_TK) {
        // activations: 32 rows x 32 k, 4 a thread; weights: 64 rows x 32 k (x 2), 8 (16) a thread
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int li = tid + i * 256, r = li >> 5, kk = li & 31;
            const int entry = rows[r];
            float v = 0.0f;
            if (entry >= 0 && k0 + kk < K) v = to_f32(A[(size_t)(GATED ? entry / top : entry) * K + k0 + kk]);
            As[kk][r] = v;
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int li = tid + i * 256, r = li >> 5, kk = li & 31;
            const bool ok = n0 + r < Nout && k0 + kk < K;
            Ws[0][kk][r] = ok ? to_f32(We[(size_t)(n0 + r) * K + k0 + kk]) : 0.0f;
            if (GATED) Ws[GATED ? 1 : 0][kk][r] = ok ? to_f32(We[(size_t)(Nout + n0 + r) * K + k0 + kk]) : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < MOE_TK; ++kk) {
            const float a0 = As[kk][ty * 2], a1 = As[kk][ty * 2 + 1];
#pragma unroll
            for (int m = 0; m < (GATED ? 2 : 1); ++m)
#pragma unroll
                for (int jn = 0; jn < 4; ++jn) {
                    const float w = Ws[m][kk][tx * 4 + jn];
                    acc[m][0][jn] = fmaf(a0, w, acc[m][0][jn]);
                    acc[m][1][jn] = fmaf(a1, w, acc[m][1][jn]);
                }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int entry = rows[ty * 2 + i];
        if (entry < 0) continue;
        const float we = wt ? wt[entry] : 1.0f;
#pragma unroll
        for (int jn = 0; jn < 4; ++jn) {
            const int n = n0 + tx * 4 + jn;
            if (n >= Nout) continue;
            if (GATED) {
                const float g = we * acc[0][i][jn], u = we * acc[GATED ? 1 : 0][i][jn];
                ((TA*)out)[(size_t)entry * Nout + n] = from_f32<TA>(act.of(g, u));
            } else {
                ((float*)out)[((size_t)(entry % top) * n_tokens + entry / top) * Nout + n] = we * acc[0][i][jn];
            }
        }
    }
}

// The same products for bfloat16 operands on the tensor cores (mma.sync m16n8k16, float32 sums):
// a tile of 16 MI entries (MI = 4, or 1 for steps with few entries an expert, whose row tiles
// would be almost empty and whose time is the tensor cores' work on the empty rows) x 64 output
// columns a block of four warps, each warp 16 of the columns (of gate and of up when GATED) for
// all rows; 64 values of k a step, staged in shared
// memory in rows of 72 values (ldmatrix then meets no bank twice), the next two steps' global
// loads in flight while the tensor cores work on this one. K must be a multiple of 8 and the operands
// 16-byte aligned (the host sees to it, else the kernel above runs).
#define MOE_MK 64
#define MOE_LD 72
template <bool GATED, int MI>
__global__ void __launch_bounds__(128)
moe_product_mma_kernel(const __nv_bfloat16* __restrict__ A, const __nv_bfloat16* __restrict__ W,
                       const int* __restrict__ sorted, const int* __restrict__ tiles, const int* __restrict__ n_tiles,
                       const float* __restrict__ wt, void* __restrict__ out, int K, int Nout, int top, int n_tokens,
                       MoeAct act) {
    constexpr int NM = GATED ? 2 : 1;
    constexpr int TM = 16 * MI;
    __shared__ __align__(16) __nv_bfloat16 As[TM * MOE_LD];
    __shared__ __align__(16) __nv_bfloat16 Ws[NM * MOE_TN * MOE_LD];
    __shared__ int rows[TM];
    pdl_trigger();
    pdl_wait();
    const int tile = blockIdx.x;
    if (tile >= *n_tiles) return;
    const int e = tiles[3 * tile], first = tiles[3 * tile + 1], cnt = tiles[3 * tile + 2];
    const int n0 = blockIdx.y * MOE_TN;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (tid < TM) rows[tid] = tid < cnt ? sorted[first + tid] : -1;
    __syncthreads();
    const __nv_bfloat16* We = W + (size_t)e * NM * Nout * K;
    // this thread's pieces of a step: MI of the activations (16 MI rows x 8 pieces of 8 values), 4
    // of each weight matrix (64 rows x 8 pieces)
    const __nv_bfloat16* a_src[MI];
    const __nv_bfloat16* w_src[NM][4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int li = tid + i * 128, r = li >> 3, c = li & 7;
        if (i < MI) {
            const int entry = rows[r];
            a_src[i] = entry >= 0 ? A + (size_t)(GATED ? entry / top : entry) * K + c * 8 : nullptr;
        }
#pragma unroll
        for (int m = 0; m < NM; ++m)
            w_src[m][i] = n0 + r < Nout ? We + ((size_t)m * Nout + n0 + r) * K + c * 8 : nullptr;
    }
    // two k steps of loads are in flight ahead of the tensor cores, in two sets of registers
    uint4 a_r0[MI], w_r0[NM][4], a_r1[MI], w_r1[NM][4];
    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
    auto fetch = [&](int k0, uint4 (&a_reg)[MI], uint4 (&w_reg)[NM][4]) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int c = (tid + i * 128) & 7;
            const bool in = k0 + c * 8 < K;
            if (i < MI) a_reg[i] = (a_src[i] && in) ? *reinterpret_cast<const uint4*>(a_src[i] + k0) : zero;
#pragma unroll
            for (int m = 0; m < NM; ++m)
                w_reg[m][i] = (w_src[m][i] && in) ? *reinterpret_cast<const uint4*>(w_src[m][i] + k0) : zero;
        }
    };
    float acc[NM][MI][2][4];
#pragma unroll
    for (int m = 0; m < NM; ++m)
#pragma unroll
        for (int mi = 0; mi < MI; ++mi)
#pragma unroll
            for (int ni = 0; ni < 2; ++ni)
#pragma unroll
                for (int x = 0; x < 4; ++x) acc[m][mi][ni][x] = 0.0f;
    // one k step: the registers' pieces go to shared memory, the registers are asked for the step
    // after the next, the tensor cores work on this one
    auto step = [&](int k0, uint4 (&a_reg)[MI], uint4 (&w_reg)[NM][4]) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int li = tid + i * 128, r = li >> 3, c = li & 7;
            if (i < MI) *reinterpret_cast<uint4*>(As + r * MOE_LD + c * 8) = a_reg[i];
#pragma unroll
            for (int m = 0; m < NM; ++m) *reinterpret_cast<uint4*>(Ws + (m * MOE_TN + r) * MOE_LD + c * 8) = w_reg[m][i];
        }
        __syncthreads();
        if (k0 + 2 * MOE_MK < K) fetch(k0 + 2 * MOE_MK, a_reg, w_reg);
#pragma unroll
        for (int kk = 0; kk < MOE_MK; kk += 16) {
            uint32_t b[NM][4];
#pragma unroll
            for (int m = 0; m < NM; ++m) {
                const int r = m * MOE_TN + warp * 16 + (lane & 7) + ((lane >> 4) << 3), c = kk + ((lane >> 3) & 1) * 8;
                ldsm_x4(b[m], smem_u32(Ws + r * MOE_LD + c));
            }
#pragma unroll
            for (int mi = 0; mi < MI; ++mi) {
                uint32_t a[4];
                ldsm_x4(a, smem_u32(As + (mi * 16 + (lane & 15)) * MOE_LD + kk + (lane >> 4) * 8));
#pragma unroll
                for (int m = 0; m < NM; ++m) {
                    mma_bf16(acc[m][mi][0], a, b[m][0], b[m][1]);
                    mma_bf16(acc[m][mi][1], a, b[m][2], b[m][3]);
                }
            }
        }
        __syncthreads();
    };
    fetch(0, a_r0, w_r0);
    if (MOE_MK < K) fetch(MOE_MK, a_r1, w_r1);
    for (int k0 = 0; k0 < K; k0 += 2 * MOE_MK) {
        step(k0, a_r0, w_r0);
        if (k0 + MOE_MK < K) step(k0 + MOE_MK, a_r1, w_r1);
    }
#pragma unroll
    for (int mi = 0; mi < MI; ++mi)
#pragma unroll
        for (int hf = 0; hf < 2; ++hf) {
            const int entry = rows[mi * 16 + (lane >> 2) + hf * 8];
            if (entry < 0) continue;
            const float we = wt ? wt[entry] : 1.0f;
#pragma unroll
            for (int ni = 0; ni < 2; ++ni)
#pragma unroll
                for (int x = 0; x < 2; ++x) {
                    const int n = n0 + warp * 16 + ni * 8 + 2 * (lane & 3) + x;
                    if (n >= Nout) continue;
                    const float v = we * acc[0][mi][ni][hf * 2 + x];
                    if (GATED) {
                        const float u = we * acc[NM - 1][mi][ni][hf * 2 + x];
                        ((__nv_bfloat16*)out)[(size_t)entry * Nout + n] = __float2bfloat16_rn(act.of(v, u));
                    } else {
                        ((float*)out)[((size_t)(entry % top) * n_tokens + entry / top) * Nout + n] = v;
                    }
                }
        }
}

// gated != 0: A [tokens, K] -> out [entries, Nout] of A's type, W [E, 2 Nout, K];
// gated == 0: A [entries, K] -> out float32 [top, tokens, Nout], W [E, Nout, K].
LUMEN_API int lumen_moe_product(const void* A, int a_is_bf16, const void* W, int w_is_bf16, const int* sorted,
                                const int* tiles, const int* n_tiles, int max_tiles, const float* wt, void* out,
                                int K, int Nout, int top, int n_tokens, int gated, int tensor_cores, int act_kind,
                                float act_limit, float act_alpha, cudaStream_t stream) {
    if (max_tiles <= 0 || n_tokens <= 0) return 0;
    if (act_kind < 0 || act_kind > 1) return LUMEN_ERR_BAD_ARGUMENT;
    const MoeAct act = {act_kind, act_limit, act_alpha};
    if (K <= 0 || Nout <= 0 || top <= 0) return LUMEN_ERR_BAD_ARGUMENT;
    dim3 grid(max_tiles, (Nout + MOE_TN - 1) / MOE_TN);
    if (grid.y > 65535) return LUMEN_ERR_UNSUPPORTED;
    if (tensor_cores) {
        // the tiles must have been made as tall as this says (lumen_moe_group): 1 tall, 2 short
        if (!a_is_bf16 || !w_is_bf16 || (K & 7) || ((uintptr_t)A & 15) || ((uintptr_t)W & 15)) return LUMEN_ERR_UNSUPPORTED;
#define MOE_MMA_GO(G_, MI_)                                                                                     \
    lumen_launch(moe_product_mma_kernel<G_, MI_>, grid, dim3(128), 0, stream, (const __nv_bfloat16*)A,          \
                 (const __nv_bfloat16*)W, sorted, tiles, n_tiles, wt, out, K, Nout, top, n_tokens, act)
        if (tensor_cores == 2) { if (gated) MOE_MMA_GO(true, 1); else MOE_MMA_GO(false, 1); }
        else { if (gated) MOE_MMA_GO(true, 4); else MOE_MMA_GO(false, 4); }
#undef MOE_MMA_GO
        LUMEN_LAUNCH_CHECK();
        return 0;
    }
#define MOE_GO(TA, TW, GATED)                                                                                        \
    lumen_launch(moe_product_kernel<TA, TW, GATED>, grid, dim3(256), 0, stream, (const TA*)A, (const TW*)W, sorted, \
                 tiles, n_tiles, wt, out, K, Nout, top, n_tokens, act)
    if (a_is_bf16 && w_is_bf16) { if (gated) MOE_GO(__nv_bfloat16, __nv_bfloat16, true); else MOE_GO(__nv_bfloat16, __nv_bfloat16, false); }
    else if (!a_is_bf16 && w_is_bf16) { if (gated) MOE_GO(float, __nv_bfloat16, true); else MOE_GO(float, __nv_bfloat16, false); }
    else if (!a_is_bf16 && !w_is_bf16) { if (gated) MOE_GO(float, float, true); else MOE_GO(float, float, false); }
    else return LUMEN_ERR_UNSUPPORTED;
#undef MOE_GO
    LUMEN_LAUNCH_CHECK();
    return 0;
}
