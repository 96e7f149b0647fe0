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
// by side), then a thread per column walks the chunks' pairs in order and leaves every chunk's
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
#pragma unroll
    for (int i = 0; i < CHUNK; ++i) {
        if (i < n) {
            const size_t row = (size_t)(t0 + i) * 3 * p.W;
            z[i] = column<TI>(p, row + c) + bz;
            u[i] = column<TI>(p, row + p.W + c) + bu;
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

// a thread per (request, column): the state every chunk starts from, and the state the portion leaves
__global__ void __launch_bounds__(NT) mingru_starts_kernel(const ScanParams p) {
    grid_launch_dependents();
    grid_dependency_wait();
    const int c = blockIdx.x * NT + threadIdx.x, b = blockIdx.z;
    if (c >= p.W) return;
    const int len = p.q_start[b + 1] - p.q_start[b];
    const int chunks = (len + CHUNK - 1) / CHUNK;
    float* st = p.state + (size_t)p.state_slot[b] * p.W + c;
    float S = p.fresh[b] ? 0.f : *st;
    const float* pr = p.pairs + (size_t)b * p.n_chunks * 2 * p.W + c;
    float* out = p.starts + (size_t)b * p.n_chunks * p.W + c;
    int j = 0;
    for (; j + 8 <= chunks; j += 8) {
        float P[8], R[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            P[i] = pr[(size_t)(j + i) * 2 * p.W];
            R[i] = pr[(size_t)(j + i) * 2 * p.W + p.W];
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            out[(size_t)(j + i) * p.W] = S;
            S = fmaf(P[i], S, R[i]);
        }
    }
    for (; j < chunks; ++j) {
        out[(size_t)j * p.W] = S;
        S = fmaf(pr[(size_t)j * 2 * p.W], S, pr[(size_t)j * 2 * p.W + p.W]);
    }
    if (chunks > 0) *st = S;
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
#pragma unroll
    for (int i = 0; i < CHUNK; ++i) {
        if (i < n) {
            const size_t row = (size_t)(t0 + i) * 3 * p.W;
            z[i] = column<TI>(p, row + c) + bz;
            u[i] = column<TI>(p, row + p.W + c) + bu;
            g[i] = column<TI>(p, row + 2 * p.W + c) + bg;
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
            if (e == cudaSuccess) e = tl_launch(mingru_starts_kernel, dim3(grid.x, 1, n_seqs), block, 0, s, p); \
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
