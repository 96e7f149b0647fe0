// Feed-forwards made of many small experts of which every token uses a few, routed on the device.
//
// route:    z = W_router x (float32; W_router may carry one more row, the shared expert's gate),
//           s = softmax(z) over the experts, the `top` experts with the largest s + correction
//           are chosen (the lower index wins a tie), their weights are s * scale (divided by their
//           sum first when renormalising); the extra row leaves as sigmoid(z).
// plan:     the (token, choice) pairs sorted by expert, stably: for every expert where its rows
//           start, the sorted order and its inverse, and the list of row tiles (expert, first
//           row, rows) that the grouped products walk.  One CTA; nothing goes back to the host,
//           so a step's launches depend on its token count only.
// grouped product:  C[r, :] = act(W[e] A[src(r), :]) for the rows r of a tile, W[e] the tile's
//           expert; float32 multiply-adds on the CUDA cores, operands float32 or bfloat16.
// combine:  out[t] = sum_k weight[t, k] * Y[place(t, k)]  (+ gate[t] * shared[t]), summed in the
//           order of the choices, so a token's result does not depend on what else is in the batch.
#include "common.cuh"
#include <math.h>

namespace {

enum : int { ACT_NONE = -1, ACT_SILU = 0, ACT_GELU_TANH = 1, ACT_RELU2 = 2 };

__device__ __forceinline__ float act_apply(float x, int act) {
    if (act == ACT_NONE) return x;
    if (act == ACT_SILU) return x / (1.f + expf(-x));
    if (act == ACT_GELU_TANH) return 0.5f * x * (1.f + tanhf(0.7978845608028654f * (x + 0.044715f * x * x * x)));
    const float r = fmaxf(x, 0.f);
    return r * r;
}

// One CTA per token.  Shared memory: the token's row as float32, then the scores.
template <typename T>
__global__ void __launch_bounds__(128) moe_route_kernel(const T* __restrict__ x, const float* __restrict__ w_router,
                                                        const float* __restrict__ correction, int* __restrict__ chosen,
                                                        float* __restrict__ weights, float* __restrict__ gate, int dim,
                                                        int n_experts, int n_rows, int top, float scale, int renormalize) {
    extern __shared__ __align__(16) float sm[];
    float* xs = sm;                 // [dim]
    float* sc = sm + dim;           // [n_rows] logits, then scores
    float* ch = sc + n_rows;        // [n_experts] what the choice looks at
    grid_launch_dependents();
    grid_dependency_wait();
    const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
    for (int d = threadIdx.x; d < dim; d += blockDim.x) xs[d] = to_float(x[(size_t)t * dim + d]);
    __syncthreads();
    for (int e = warp; e < n_rows; e += n_warps) {
        const float* wr = w_router + (size_t)e * dim;
        float acc = 0.f;
        for (int d = lane; d < dim; d += 32) acc = fmaf(xs[d], wr[d], acc);
        acc = warp_sum(acc);
        if (lane == 0) sc[e] = acc;
    }
    __syncthreads();
    if (warp != 0) return;
    float mx = -INFINITY;
    for (int e = lane; e < n_experts; e += 32) mx = fmaxf(mx, sc[e]);
    mx = warp_max(mx);
    float sum = 0.f;
    for (int e = lane; e < n_experts; e += 32) sum += expf(sc[e] - mx);
    sum = warp_sum(sum);
    const float inv = 1.f / sum;
    for (int e = lane; e < n_experts; e += 32) {
        const float s = expf(sc[e] - mx) * inv;
        sc[e] = s;
        ch[e] = s + (correction != nullptr ? correction[e] : 0.f);
    }
    if (lane == 0 && gate != nullptr) gate[t] = 1.f / (1.f + expf(-sc[n_experts]));
    __syncwarp();
    float total = 0.f;
    for (int k = 0; k < top; ++k) {
        float best = -INFINITY;
        int at = 0x7fffffff;
        for (int e = lane; e < n_experts; e += 32) {
            const float v = ch[e];
            if (v > best) { best = v; at = e; }       // (a lane walks upwards: the lower index stays on a tie)
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oa = __shfl_xor_sync(0xffffffffu, at, o);
            if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; }
        }
        if (at >= n_experts) at = 0;                  // (all scores NaN: stay in bounds)
        if (lane == 0) {
            chosen[(size_t)t * top + k] = at;
            weights[(size_t)t * top + k] = sc[at];
            ch[at] = -INFINITY;
        }
        total += sc[at];
        __syncwarp();
    }
    if (lane == 0) {
        const float f = renormalize ? scale / total : scale;
        for (int k = 0; k < top; ++k) weights[(size_t)t * top + k] *= f;
    }
}

// One CTA.  counts/offsets live in shared memory ([n_experts + 1] ints each).
__global__ void __launch_bounds__(1024) moe_plan_kernel(const int* __restrict__ chosen, int n_pairs, int n_experts, int tile_rows,
                                                        int* __restrict__ order, int* __restrict__ place,
                                                        int* __restrict__ tiles, int max_tiles) {
    extern __shared__ int ism[];
    int* counts = ism;                    // [n_experts]
    int* offsets = ism + n_experts;       // [n_experts + 1]
    grid_launch_dependents();
    grid_dependency_wait();
    for (int e = threadIdx.x; e < n_experts; e += blockDim.x) counts[e] = 0;
    __syncthreads();
    for (int a = threadIdx.x; a < n_pairs; a += blockDim.x) {
        const int e = chosen[a];
        if (e >= 0 && e < n_experts) atomicAdd(&counts[e], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int off = 0, n_tiles = 0;
        for (int e = 0; e < n_experts; ++e) {
            offsets[e] = off;
            for (int r = 0; r < counts[e] && n_tiles < max_tiles; r += tile_rows) {
                tiles[1 + 3 * n_tiles] = e;
                tiles[2 + 3 * n_tiles] = off + r;
                tiles[3 + 3 * n_tiles] = min(tile_rows, counts[e] - r);
                ++n_tiles;
            }
            off += counts[e];
        }
        offsets[n_experts] = off;
        tiles[0] = n_tiles;
    }
    __syncthreads();
    // stable placement: a warp per expert walks the pairs in order
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
    for (int e = warp; e < n_experts; e += n_warps) {
        if (counts[e] == 0) continue;
        int at = offsets[e];
        for (int a0 = 0; a0 < n_pairs; a0 += 32) {
            const int a = a0 + lane;
            const bool mine = a < n_pairs && chosen[a] == e;
            const unsigned m = __ballot_sync(0xffffffffu, mine);
            if (mine) {
                const int pos = at + __popc(m & ((1u << lane) - 1u));
                order[pos] = a;
                place[a] = pos;
            }
            at += __popc(m);
        }
    }
}

constexpr int BN = 64, BK = 16, PAD = 4, NT = 256;

// grid: (N slabs, tiles).  BM rows of one expert per CTA (16 or 64), 64 columns, K walked 16 at a time.
template <typename T, typename TO, int BM>
__global__ void __launch_bounds__(NT) moe_gemm_kernel(const T* __restrict__ A, const T* __restrict__ W, TO* __restrict__ C,
                                                      const int* __restrict__ tiles, const int* __restrict__ order,
                                                      int gather_div, int N, int K, int act) {
    constexpr int TM = BM / 16;
    __shared__ float As[BK][BM + PAD];
    __shared__ float Ws[BK][BN + PAD];
    __shared__ int src[BM];
    grid_launch_dependents();
    grid_dependency_wait();
    const int tile = blockIdx.y;
    if (tile >= tiles[0]) return;
    const int e = tiles[1 + 3 * tile], row0 = tiles[2 + 3 * tile], n_rows = tiles[3 + 3 * tile];
    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    const int n0 = blockIdx.x * BN;
    for (int r = tid; r < BM; r += NT) src[r] = r < n_rows ? (gather_div > 0 ? order[row0 + r] / gather_div : row0 + r) : -1;
    __syncthreads();
    W += (size_t)e * N * K;
    const int lrow = tid >> 2, lk = (tid & 3) * 4;       // loads: a row (of 64) and four k
    float acc[TM][4];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
    for (int k0 = 0; k0 < K; k0 += BK) {
        const int gn = n0 + lrow;
        const int srow = lrow < BM ? src[lrow] : -1;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const int gk = k0 + lk + q;
            if (lrow < BM) As[lk + q][lrow] = (srow >= 0 && gk < K) ? to_float(A[(size_t)srow * K + gk]) : 0.f;
            Ws[lk + q][lrow] = (gn < N && gk < K) ? to_float(W[(size_t)gn * K + gk]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < BK; ++k) {
            const float4 w4 = *reinterpret_cast<const float4*>(&Ws[k][tx * 4]);
            const float w[4] = {w4.x, w4.y, w4.z, w4.w};
#pragma unroll
            for (int i = 0; i < TM; ++i) {
                const float a = As[k][ty * TM + i];
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a, w[j], acc[i][j]);
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int r = ty * TM + i;
        if (r >= n_rows) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int gn = n0 + tx * 4 + j;
            if (gn < N) C[(size_t)(row0 + r) * N + gn] = from_float<TO>(act_apply(acc[i][j], act));
        }
    }
}

// One CTA per token.  y: [pairs][dim] in sorted order; shared: [splits][T][dim] or null.
template <typename T, typename TS>
__global__ void moe_combine_kernel(const T* __restrict__ y, const int* __restrict__ place, const float* __restrict__ weights,
                                   const TS* __restrict__ shared, int shared_splits, long long shared_plane,
                                   const float* __restrict__ gate, T* __restrict__ out, int dim, int top) {
    grid_launch_dependents();
    grid_dependency_wait();
    const int t = blockIdx.x;
    for (int d = threadIdx.x; d < dim; d += blockDim.x) {
        float acc = 0.f;
        for (int k = 0; k < top; ++k)
            acc = fmaf(weights[(size_t)t * top + k], to_float(y[(size_t)place[(size_t)t * top + k] * dim + d]), acc);
        if (shared != nullptr) {
            float sh = 0.f;
            for (int s = 0; s < shared_splits; ++s) sh += to_float(shared[(size_t)s * shared_plane + (size_t)t * dim + d]);
            acc = gate != nullptr ? fmaf(gate[t], sh, acc) : acc + sh;
        }
        out[(size_t)t * dim + d] = from_float<T>(acc);
    }
}

}  // namespace

// x: [n_tokens][dim] of dtype; w_router: float32 [n_rows][dim], n_rows = n_experts (+ 1 with gate != null);
// correction: float32 [n_experts] or null; chosen: int32 [n_tokens][top]; weights: float32 [n_tokens][top];
// gate: float32 [n_tokens] or null.
extern "C" int tl_moe_route(const void* x, int dtype, const float* w_router, const float* correction, int* chosen,
                            float* weights, float* gate, int n_tokens, int dim, int n_experts, int top, float scale,
                            int renormalize, void* stream) {
    if (n_tokens <= 0) return TL_OK;
    if (dim <= 0 || n_experts <= 0 || top <= 0 || top > n_experts) return TL_BAD_SIZE;
    const int n_rows = n_experts + (gate != nullptr ? 1 : 0);
    const size_t smem = (size_t)(dim + n_rows + n_experts) * sizeof(float);
    if (smem > 48 * 1024) return TL_TOO_LARGE;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == TL_F32)
        return (int)tl_launch(moe_route_kernel<float>, dim3(n_tokens), dim3(128), smem, s, (const float*)x, w_router, correction,
                              chosen, weights, gate, dim, n_experts, n_rows, top, scale, renormalize);
    if (dtype == TL_BF16)
        return (int)tl_launch(moe_route_kernel<__nv_bfloat16>, dim3(n_tokens), dim3(128), smem, s, (const __nv_bfloat16*)x, w_router,
                              correction, chosen, weights, gate, dim, n_experts, n_rows, top, scale, renormalize);
    return TL_BAD_DTYPE;
}

// rows of a tile for this many (token, choice) pairs, and how many tiles there can be at most
extern "C" int tl_moe_tile_rows(int n_pairs) { return n_pairs <= 512 ? 16 : 64; }
extern "C" int tl_moe_max_tiles(int n_pairs, int n_experts) {
    const int rows = tl_moe_tile_rows(n_pairs);
    const long long most = (long long)(n_pairs + rows - 1) / rows + n_experts;
    return (int)(most < n_pairs ? most : n_pairs);
}

// chosen: int32 [n_pairs]; order, place: int32 [n_pairs]; tiles: int32 [1 + 3 * max_tiles] (count, then
// expert, first row, rows of every tile)
extern "C" int tl_moe_plan(const int* chosen, int n_pairs, int n_experts, int* order, int* place, int* tiles, void* stream) {
    if (n_pairs <= 0) return TL_OK;
    if (n_experts <= 0 || n_experts > 4096) return TL_BAD_SIZE;
    const size_t smem = (size_t)(2 * n_experts + 1) * sizeof(int);
    return (int)tl_launch(moe_plan_kernel, dim3(1), dim3(1024), smem, (cudaStream_t)stream, chosen, n_pairs, n_experts,
                          tl_moe_tile_rows(n_pairs), order, place, tiles, tl_moe_max_tiles(n_pairs, n_experts));
}

// The experts' products over the sorted rows.  A: [rows][K]; with gather_div > 0 row r of the sorted order
// reads A[order[r] / gather_div] (a token's row for each of its choices), else A[r].  W: [n_experts][N][K];
// C: [n_pairs][N] in sorted order.  act: -1 none, 0 silu, 1 gelu (tanh form), 2 squared relu.
extern "C" int tl_moe_gemm(const void* A, const void* W, void* C, int dtype, const int* tiles, const int* order,
                           int gather_div, int n_pairs, int n_experts, int N, int K, int act, void* stream) {
    if (n_pairs <= 0 || N <= 0) return TL_OK;
    if (K <= 0 || act < -1 || act > 2) return TL_BAD_SIZE;
    const int max_tiles = tl_moe_max_tiles(n_pairs, n_experts);
    if (max_tiles > 65535) return TL_BAD_SIZE;
    const dim3 grid((N + BN - 1) / BN, max_tiles), block(NT);
    cudaStream_t s = (cudaStream_t)stream;
    const bool small = tl_moe_tile_rows(n_pairs) == 16;
#define TL_MOE_GEMM(T, BM) \
    tl_launch(moe_gemm_kernel<T, T, BM>, grid, block, 0, s, (const T*)A, (const T*)W, (T*)C, tiles, order, gather_div, N, K, act)
    if (dtype == TL_F32) return (int)(small ? TL_MOE_GEMM(float, 16) : TL_MOE_GEMM(float, 64));
    if (dtype == TL_BF16) return (int)(small ? TL_MOE_GEMM(__nv_bfloat16, 16) : TL_MOE_GEMM(__nv_bfloat16, 64));
#undef TL_MOE_GEMM
    return TL_BAD_DTYPE;
}

// y: [n_tokens * top][dim] of dtype in sorted order; shared: [shared_splits][n_tokens][dim] of shared_dtype or
// null; gate: float32 [n_tokens] or null; out: [n_tokens][dim] of dtype.
extern "C" int tl_moe_combine(const void* y, int dtype, const int* place, const float* weights, const void* shared,
                              int shared_dtype, int shared_splits, long long shared_plane, const float* gate, void* out,
                              int n_tokens, int dim, int top, void* stream) {
    if (n_tokens <= 0) return TL_OK;
    if (dim <= 0 || top <= 0) return TL_BAD_SIZE;
    const dim3 grid(n_tokens), block(dim >= 1024 ? 256 : 128);
    cudaStream_t s = (cudaStream_t)stream;
#define TL_MOE_COMBINE(T, TS)                                                                                       \
    tl_launch(moe_combine_kernel<T, TS>, grid, block, 0, s, (const T*)y, place, weights, (const TS*)shared, shared_splits, \
              shared_plane, gate, (T*)out, dim, top)
    if (dtype == TL_F32 && (shared == nullptr || shared_dtype == TL_F32)) return (int)TL_MOE_COMBINE(float, float);
    if (dtype == TL_BF16 && (shared == nullptr || shared_dtype == TL_BF16)) return (int)TL_MOE_COMBINE(__nv_bfloat16, __nv_bfloat16);
    if (dtype == TL_BF16 && shared_dtype == TL_F32) return (int)TL_MOE_COMBINE(__nv_bfloat16, float);
#undef TL_MOE_COMBINE
    return TL_BAD_DTYPE;
}
