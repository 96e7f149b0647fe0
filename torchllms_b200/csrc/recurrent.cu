// Recurrences with a state of fixed size per request.
//
// mingru_scan: a gated recurrence whose gates read the current token only.  A token's row of the
// stacked projection is [z | u | g], W columns each (a bias is added first):
//     a = sigmoid(z);   c = u + 1/2 where u >= 0, sigmoid(u) elsewhere;
//     S <- (1 - a) S + a c      (element by element; S is the request's state row, float32)
//     out = S * g * sigmoid(g)
// Everything is float32 arithmetic; the projection may arrive as bfloat16 or as float32 partial
// sums of a split-K product, the result leaves in the activation dtype.
//
// A request's portion is a linear recurrence S_t = p_t S_(t-1) + r_t, so it can be cut into chunks:
// every chunk first reduces to the pair (P, R) with S_end = P S_start + R (kernel 1, all chunks side
// by side), then the chunks' pairs are walked in order, in two levels, which leaves every chunk's
// S_start and the request's new state (kernel 2), then every chunk runs its tokens again from its
// S_start, writing the outputs (kernel 3).  Portions no longer than one chunk (decode steps among
// them) run as kernel 3 alone.  A thread owns one column of one chunk and fetches the chunk's
// values before it starts on the recurrence, so reads are side by side along the row and many are
// in flight.
#include "common.cuh"

namespace {

constexpr int CHUNK = 8;      // tokens a thread walks in one go
constexpr int NT = 128;

struct ScanParams {
    const void* proj;        // [splits][T][3 W]
    int splits;
    long long plane;
    const float* bias;       // [3 W] or null
    float* state;            // [slots][W]
    const int* q_start;      // [B + 1]
    const int* state_slot;   // [B]
    const int* fresh;        // [B]: 1 where the request starts here (its state counts as zero)
    void* out;               // [T][W]
    float* pairs;            // [B][n_chunks][2][W]: P and R of every chunk
    float* starts;           // [B][n_chunks][W]: the state every chunk starts from
    int W, n_chunks;
};

template <typename TI>
__device__ __forceinline__ float column(const ScanParams& p, size_t at) {
    const TI* src = reinterpret_cast<const TI*>(p.proj);
    float x = to_float(src[at]);
    for (int s = 1; s < p.splits; ++s) x += to_float(src[(size_t)s * p.plane + at]);
    return x;
}

// FAST (results that leave as bfloat16): the hardware's exponential and reciprocal, good to a few units in the
// last place of float32; the float32 mode takes the library's.
template <bool FAST>
__device__ __forceinline__ float sigmoidf_(float x) {
    return FAST ? __fdividef(1.f, 1.f + __expf(-x)) : 1.f / (1.f + expf(-x));
}

// S <- keep * S + add from a token's z and u columns (biases added)
template <bool FAST>
__device__ __forceinline__ void token_terms(float z, float u, float& keep, float& add) {
    const float a = sigmoidf_<FAST>(z);
    const float cand = u >= 0.f ? u + 0.5f : sigmoidf_<FAST>(u);
    keep = 1.f - a;
    add = a * cand;
}

template <typename TI, bool FAST>
__global__ void __launch_bounds__(NT, 8) mingru_pairs_kernel(const ScanParams p) {
    grid_launch_dependents();
    grid_dependency_wait();
    const int c = blockIdx.x * NT + threadIdx.x;
    const int chunk = blockIdx.y, b = blockIdx.z;
    if (c >= p.W) return;
    const int t0 = p.q_start[b] + chunk * CHUNK, n = min(p.q_start[b + 1] - t0, CHUNK);
    if (n <= 0) return;
    const float bz = p.bias ? p.bias[c] : 0.f, bu = p.bias ? p.bias[p.W + c] : 0.f;
    float z[CHUNK], u[CHUNK];
    if (p.splits == 1) {
        // one plane (prompt portions): every load is issued before anything waits for one; a short last chunk
        // fetches its last token again in place of the absent ones
        const TI* src = reinterpret_cast<const TI*>(p.proj);
#pragma unroll
        for (int i = 0; i < CHUNK; ++i) {
            const size_t row = (size_t)(t0 + min(i, n - 1)) * 3 * p.W;
            z[i] = to_float(src[row + c]);
            u[i] = to_float(src[row + p.W + c]);
        }
#pragma unroll
        for (int i = 0; i < CHUNK; ++i) {
            z[i] += bz;
            u[i] += bu;
        }
    } else {
#pragma unroll
        for (int i = 0; i < CHUNK; ++i) {
            if (i < n) {
                const size_t row = (size_t)(t0 + i) * 3 * p.W;
                z[i] = column<TI>(p, row + c) + bz;
                u[i] = column<TI>(p, row + p.W + c) + bu;
            }
        }
    }
    float P = 1.f, R = 0.f;
#pragma unroll
    for (int i = 0; i < CHUNK; ++i) {
        if (i < n) {
            float keep, add;
            token_terms<FAST>(z[i], u[i], keep, add);
            P *= keep;
            R = fmaf(keep, R, add);
        }
    }
    float* pr = p.pairs + ((size_t)b * p.n_chunks + chunk) * 2 * p.W;
    pr[c] = P;
    pr[p.W + c] = R;
}

// The state every chunk starts from, and the state the portion leaves.  A CTA per (request, 32 columns): its
// eight warps each take an eighth of the chunks, fold their pairs into one, learn their own start from the
// warps before them, and walk their chunks again.  A lane is a column, so rows are read side by side.
constexpr int SW = 8;         // warps of the starts kernel
__global__ void __launch_bounds__(32 * SW) mingru_starts_kernel(const ScanParams p) {
    __shared__ float sP[SW][32], sR[SW][32];
    grid_launch_dependents();
    grid_dependency_wait();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int c = blockIdx.x * 32 + lane, b = blockIdx.z;
    const bool live = c < p.W;
    const int cc = live ? c : p.W - 1;
    const int len = p.q_start[b + 1] - p.q_start[b];
    const int chunks = (len + CHUNK - 1) / CHUNK;
    const int per = (chunks + SW - 1) / SW;
    const int j0 = min(warp * per, chunks), j1 = min(j0 + per, chunks);
    const float* pr = p.pairs + (size_t)b * p.n_chunks * 2 * p.W + cc;
    float P = 1.f, R = 0.f;
    for (int j = j0; j < j1; j += 8) {
        float Pj[8], Rj[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const size_t at = (size_t)min(j + i, j1 - 1) * 2 * p.W;
            Pj[i] = pr[at];
            Rj[i] = pr[at + p.W];
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            if (j + i < j1) {
                R = fmaf(Pj[i], R, Rj[i]);
                P *= Pj[i];
            }
        }
    }
    sP[warp][lane] = P;
    sR[warp][lane] = R;
    __syncthreads();
    float* st = p.state + (size_t)p.state_slot[b] * p.W + cc;
    float S = p.fresh[b] ? 0.f : *st;
    for (int w = 0; w < warp; ++w) S = fmaf(sP[w][lane], S, sR[w][lane]);
    float* out = p.starts + (size_t)b * p.n_chunks * p.W + cc;
    for (int j = j0; j < j1; j += 8) {
        float Pj[8], Rj[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const size_t at = (size_t)min(j + i, j1 - 1) * 2 * p.W;
            Pj[i] = pr[at];
            Rj[i] = pr[at + p.W];
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            if (j + i < j1) {
                if (live) out[(size_t)(j + i) * p.W] = S;
                S = fmaf(Pj[i], S, Rj[i]);
            }
        }
    }
    __syncthreads();                                       // every warp has read the state it started from
    if (live && j0 < j1 && j1 == chunks) *st = S;          // the warp that owns the last chunk leaves the state
}

template <typename TI, typename TO, bool FAST>
__global__ void __launch_bounds__(NT, 8) mingru_scan_kernel(const ScanParams p) {
    grid_launch_dependents();
    grid_dependency_wait();
    const int c = blockIdx.x * NT + threadIdx.x;
    const int chunk = blockIdx.y, b = blockIdx.z;
    if (c >= p.W) return;
    const int t0 = p.q_start[b] + chunk * CHUNK, n = min(p.q_start[b + 1] - t0, CHUNK);
    if (n <= 0) return;
    const float bz = p.bias ? p.bias[c] : 0.f, bu = p.bias ? p.bias[p.W + c] : 0.f, bg = p.bias ? p.bias[2 * p.W + c] : 0.f;
    float z[CHUNK], u[CHUNK], g[CHUNK];
    if (p.splits == 1 && n > 1) {
        const TI* src = reinterpret_cast<const TI*>(p.proj);      // (as in the kernel above)
#pragma unroll
        for (int i = 0; i < CHUNK; ++i) {
            const size_t row = (size_t)(t0 + min(i, n - 1)) * 3 * p.W;
            z[i] = to_float(src[row + c]);
            u[i] = to_float(src[row + p.W + c]);
            g[i] = to_float(src[row + 2 * p.W + c]);
        }
#pragma unroll
        for (int i = 0; i < CHUNK; ++i) {
            z[i] += bz;
            u[i] += bu;
            g[i] += bg;
        }
    } else {
#pragma unroll
        for (int i = 0; i < CHUNK; ++i) {
            if (i < n) {
                const size_t row = (size_t)(t0 + i) * 3 * p.W;
                z[i] = column<TI>(p, row + c) + bz;
                u[i] = column<TI>(p, row + p.W + c) + bu;
                g[i] = column<TI>(p, row + 2 * p.W + c) + bg;
            }
        }
    }
    float* st = p.state + (size_t)p.state_slot[b] * p.W + c;
    float S = p.n_chunks == 1 ? (p.fresh[b] ? 0.f : *st) : p.starts[((size_t)b * p.n_chunks + chunk) * p.W + c];
    TO* out = reinterpret_cast<TO*>(p.out);
#pragma unroll
    for (int i = 0; i < CHUNK; ++i) {
        if (i < n) {
            float keep, add;
            token_terms<FAST>(z[i], u[i], keep, add);
            S = fmaf(keep, S, add);
            out[(size_t)(t0 + i) * p.W + c] = from_float<TO>(S * g[i] * sigmoidf_<FAST>(g[i]));
        }
    }
    if (p.n_chunks == 1) *st = S;     // (longer portions: the walk over the chunks left the state)
}

}  // namespace

// float32 words of scratch that a call with these sizes needs (0: none)
extern "C" long long tl_mingru_scan_scratch(int n_seqs, int width, int max_q_len) {
    const long long n_chunks = (max_q_len + CHUNK - 1) / CHUNK;
    return n_chunks <= 1 ? 0 : (long long)n_seqs * width * 3 * n_chunks;
}

// proj: [splits][n_tokens][3 * width] of in_dtype; bias: float32 [3 * width] or null; state: float32
// [slots][width]; out: [n_tokens][width] of out_dtype; scratch: as tl_mingru_scan_scratch says.
extern "C" int tl_mingru_scan(const void* proj, int in_dtype, int splits, long long plane, const float* bias, float* state,
                              const int* q_start, const int* state_slot, const int* fresh, void* out, int out_dtype,
                              int n_tokens, int n_seqs, int width, int max_q_len, float* scratch, void* stream) {
    if (n_tokens <= 0 || n_seqs <= 0) return TL_OK;
    if (width <= 0 || max_q_len <= 0 || splits < 1 || n_seqs > 65535) return TL_BAD_SIZE;
    ScanParams p;
    p.proj = proj; p.splits = splits; p.plane = plane; p.bias = bias; p.state = state;
    p.q_start = q_start; p.state_slot = state_slot; p.fresh = fresh; p.out = out;
    p.W = width;
    p.n_chunks = (max_q_len + CHUNK - 1) / CHUNK;
    if (p.n_chunks > 65535) return TL_BAD_SIZE;
    if (p.n_chunks > 1 && scratch == nullptr) return TL_BAD_SIZE;
    p.pairs = scratch;
    p.starts = scratch ? scratch + (size_t)n_seqs * width * 2 * p.n_chunks : nullptr;
    cudaStream_t s = (cudaStream_t)stream;
    const dim3 grid((width + NT - 1) / NT, p.n_chunks, n_seqs), block(NT);
    cudaError_t e = cudaSuccess;
#define TL_SCAN(TI, TO, FAST)                                                                          \
    do {                                                                                         \
        if (p.n_chunks > 1) {                                                                    \
            e = tl_launch(mingru_pairs_kernel<TI, FAST>, grid, block, 0, s, p);                  \
            if (e == cudaSuccess) e = tl_launch(mingru_starts_kernel, dim3((width + 31) / 32, 1, n_seqs), dim3(32 * SW), 0, s, p); \
        }                                                                                        \
        if (e == cudaSuccess) e = tl_launch(mingru_scan_kernel<TI, TO, FAST>, grid, block, 0, s, p); \
    } while (0)
    if (in_dtype == TL_F32 && out_dtype == TL_F32) TL_SCAN(float, float, false);
    else if (in_dtype == TL_F32 && out_dtype == TL_BF16) TL_SCAN(float, __nv_bfloat16, true);
    else if (in_dtype == TL_BF16 && out_dtype == TL_BF16) TL_SCAN(__nv_bfloat16, __nv_bfloat16, true);
    else return TL_BAD_DTYPE;
#undef TL_SCAN
    return (int)e;
}
