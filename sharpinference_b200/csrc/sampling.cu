// Choosing the next token on the device: greedy argmax, and temperature sampling with the
// reference's filters in the reference's order (src/SharpInference.Engine/Sampler.cs:15-107):
// logit bias and window penalties in logit space, temperature, softmax, top-k (+ renormalise),
// min-p, top-p, renormalise, inverse-CDF draw (first index whose cumulative mass reaches the
// uniform number, :564-576).  Greedy takes the lowest index among equal maxima (:436-449; the
// reference's device argmax keeps the same rule, src/SharpInference.Cuda/CudaTextKernels.cs:393-402).
//
// One block handles one row.  The uniform number comes from the caller (a counter-based
// generator keyed by the request's seed), so a request draws the same tokens whatever else is
// in the batch.
#include "common.cuh"

constexpr int SAMPLE_THREADS = 1024;

struct ArgBest {
    float v;
    int i;
};

__device__ __forceinline__ ArgBest better(ArgBest a, ArgBest b) {
    if (b.v > a.v || (b.v == a.v && b.i < a.i)) return b;
    return a;
}

// Largest value with the lowest index among ties, over the whole block.
__device__ ArgBest block_argmax(ArgBest mine, ArgBest* scratch /*[32]*/) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = (blockDim.x + 31) >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        ArgBest other;
        other.v = __shfl_xor_sync(0xffffffffu, mine.v, o);
        other.i = __shfl_xor_sync(0xffffffffu, mine.i, o);
        mine = better(mine, other);
    }
    __syncthreads();
    if (lane == 0) scratch[warp] = mine;
    __syncthreads();
    ArgBest r;
    r.v = -INFINITY;
    r.i = 0x7fffffff;
    if (lane < nwarps) r = scratch[lane];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        ArgBest other;
        other.v = __shfl_xor_sync(0xffffffffu, r.v, o);
        other.i = __shfl_xor_sync(0xffffffffu, r.i, o);
        r = better(r, other);
    }
    return r;
}

__device__ int row_argmax(const float* __restrict__ row, int V, ArgBest* scratch) {
    ArgBest mine;
    mine.v = -INFINITY;
    mine.i = 0x7fffffff;
    if ((V % 4 == 0) && ((reinterpret_cast<uintptr_t>(row) & 15) == 0)) {
        const float4* row4 = reinterpret_cast<const float4*>(row);
        for (int i = threadIdx.x; i < V / 4; i += blockDim.x) {   // ascending indices per thread
            const float4 v = row4[i];
            if (v.x > mine.v) { mine.v = v.x; mine.i = 4 * i; }
            if (v.y > mine.v) { mine.v = v.y; mine.i = 4 * i + 1; }
            if (v.z > mine.v) { mine.v = v.z; mine.i = 4 * i + 2; }
            if (v.w > mine.v) { mine.v = v.w; mine.i = 4 * i + 3; }
        }
    } else {
        for (int i = threadIdx.x; i < V; i += blockDim.x) {
            const float v = row[i];
            if (v > mine.v) {  // ascending i per thread: strict > keeps the lowest index
                mine.v = v;
                mine.i = i;
            }
        }
    }
    ArgBest r = block_argmax(mine, scratch);
    return r.i == 0x7fffffff ? 0 : r.i;  // all -inf or NaN: index 0, as a left-to-right scan gives
}

__global__ void argmax_rows_kernel(const float* __restrict__ logits, int V, int* __restrict__ out) {
    __shared__ ArgBest scratch[32];
    pdl_wait();
    const int r = blockIdx.x;
    const int best = row_argmax(logits + (size_t)r * V, V, scratch);
    if (threadIdx.x == 0) out[r] = best;
}

// Few rows: one block per row would leave the GPU to a handful of blocks that wait for memory.  Then a row
// is cut into ARGMAX_SLICES slices with a block each; the block that finishes last for a row (a ticket,
// left at zero again) picks among the slices' candidates.  Ties still go to the lowest index.
constexpr int ARGMAX_SLICES = 32;

__global__ void argmax_rows_sliced_kernel(const float* __restrict__ logits, int V, int* __restrict__ out,
                                          ArgBest* __restrict__ cand, int* __restrict__ tickets) {
    __shared__ ArgBest scratch[32];
    __shared__ int last_s;
    pdl_wait();
    const int r = blockIdx.y, sl = blockIdx.x;
    const int per = (((V + ARGMAX_SLICES - 1) / ARGMAX_SLICES) + 3) & ~3;
    const int begin = min(V, sl * per), end = min(V, begin + per);
    const float* row = logits + (size_t)r * V;
    ArgBest mine;
    mine.v = -INFINITY;
    mine.i = 0x7fffffff;
    for (int i = begin + threadIdx.x; i < end; i += blockDim.x) {
        const float v = row[i];
        if (v > mine.v) {  // ascending i per thread: strict > keeps the lowest index
            mine.v = v;
            mine.i = i;
        }
    }
    const ArgBest best = block_argmax(mine, scratch);
    if (threadIdx.x == 0) {
        cand[(size_t)r * ARGMAX_SLICES + sl] = best;
        __threadfence();
        last_s = (atomicAdd(&tickets[r], 1) == ARGMAX_SLICES - 1);
        if (last_s) tickets[r] = 0;
    }
    __syncthreads();
    if (!last_s) return;
    __threadfence();
    ArgBest c;
    c.v = -INFINITY;
    c.i = 0x7fffffff;
    if (threadIdx.x < ARGMAX_SLICES) {
        const ArgBest* p = cand + (size_t)r * ARGMAX_SLICES + threadIdx.x;
        c.v = __ldcg(&p->v);
        c.i = __ldcg(&p->i);
    }
    const ArgBest all = block_argmax(c, scratch);
    if (threadIdx.x == 0) out[r] = all.i == 0x7fffffff ? 0 : all.i;
}

// `scratch` (optional): 64 ints that are zero before the call (and after it), then 64 * 32 pairs of (float, int);
// with it, calls for up to 16 rows cut every row over 32 blocks.
SHARPI_API int sharpi_argmax_rows(const float* logits, int R, int V, int* out, void* scratch, cudaStream_t stream) {
    if (R <= 0) return SHARPI_OK;
    if (V <= 0) return SHARPI_BAD_ARGUMENT;
    if (scratch && R <= 16 && V >= 4096) {      // more rows fill the GPU with a block each
        int* tickets = reinterpret_cast<int*>(scratch);
        ArgBest* cand = reinterpret_cast<ArgBest*>(tickets + 64);
        SHARPI_LAUNCH_PDL(argmax_rows_sliced_kernel, dim3(ARGMAX_SLICES, R), SAMPLE_THREADS, 0, stream, logits, V, out, cand,
                          tickets);
        return SHARPI_OK;
    }
    SHARPI_LAUNCH_PDL(argmax_rows_kernel, R, SAMPLE_THREADS, 0, stream, logits, V, out);
    return SHARPI_OK;
}

// ---------------------------------------------------------------------------------------
// Sparse edits of the logits before sampling.  Every (row, token) pair occurs at most once.
// ---------------------------------------------------------------------------------------
__global__ void apply_penalties_kernel(float* __restrict__ logits, int V, const int* __restrict__ entry_row,
                                       const int* __restrict__ entry_token, const int* __restrict__ entry_count,
                                       const float* __restrict__ rep, const float* __restrict__ freq,
                                       const float* __restrict__ pres, int N) {
    const int n = blockIdx.x * blockDim.x + threadIdx.x;
    if (n >= N) return;
    const int r = entry_row[n], id = entry_token[n];
    if (id < 0 || id >= V) return;
    float v = logits[(size_t)r * V + id];
    const float rp = rep[r];
    if (rp != 1.0f) v = v > 0.0f ? v / rp : v * rp;
    if (freq[r] != 0.0f || pres[r] != 0.0f) v -= (float)entry_count[n] * freq[r] + pres[r];
    logits[(size_t)r * V + id] = v;
}

SHARPI_API int sharpi_apply_penalties(float* logits, int V, const int* entry_row, const int* entry_token,
                                      const int* entry_count, const float* rep, const float* freq,
                                      const float* pres, int N, cudaStream_t stream) {
    if (N <= 0) return SHARPI_OK;
    apply_penalties_kernel<<<(N + 255) / 256, 256, 0, stream>>>(logits, V, entry_row, entry_token, entry_count,
                                                                rep, freq, pres, N);
    SHARPI_CHECK_LAUNCH();
    return SHARPI_OK;
}

__global__ void add_logit_bias_kernel(float* __restrict__ logits, int V, const int* __restrict__ entry_row,
                                      const int* __restrict__ entry_token, const float* __restrict__ entry_bias,
                                      int N) {
    const int n = blockIdx.x * blockDim.x + threadIdx.x;
    if (n >= N) return;
    const int id = entry_token[n];
    if (id < 0 || id >= V) return;
    logits[(size_t)entry_row[n] * V + id] += entry_bias[n];
}

SHARPI_API int sharpi_add_logit_bias(float* logits, int V, const int* entry_row, const int* entry_token,
                                     const float* entry_bias, int N, cudaStream_t stream) {
    if (N <= 0) return SHARPI_OK;
    add_logit_bias_kernel<<<(N + 255) / 256, 256, 0, stream>>>(logits, V, entry_row, entry_token, entry_bias, N);
    SHARPI_CHECK_LAUNCH();
    return SHARPI_OK;
}

// ---------------------------------------------------------------------------------------
// Temperature sampling with top-k / min-p / top-p.  `probs` is caller-provided scratch [R, V].
// ---------------------------------------------------------------------------------------
__device__ void normalize_row(float* __restrict__ p, int V, float* scratch) {
    float s = 0.0f;
    for (int i = threadIdx.x; i < V; i += SAMPLE_THREADS) s += p[i];
    s = block_sum(s, scratch);
    if (s > 0.0f && s != 1.0f) {
        const float inv = 1.0f / s;
        for (int i = threadIdx.x; i < V; i += SAMPLE_THREADS) p[i] *= inv;
    }
    __syncthreads();
}

__global__ void sample_rows_kernel(const float* __restrict__ logits, int V, const float* __restrict__ temperature,
                                   const int* __restrict__ top_k, const float* __restrict__ top_p,
                                   const float* __restrict__ min_p, const float* __restrict__ uniform,
                                   float* __restrict__ probs, int* __restrict__ out) {
    __shared__ float scratch[32];
    __shared__ ArgBest ascratch[32];
    __shared__ float prefix_s[SAMPLE_THREADS];
    __shared__ int pick_s;

    const int r = blockIdx.x;
    const float* row = logits + (size_t)r * V;
    const float temp = temperature[r];
    if (temp <= 0.0f) {
        const int best = row_argmax(row, V, ascratch);
        if (threadIdx.x == 0) out[r] = best;
        return;
    }
    float* p = probs + (size_t)r * V;
    const float inv_t = 1.0f / temp;

    // softmax(logits / T)
    float m = -INFINITY;
    for (int i = threadIdx.x; i < V; i += SAMPLE_THREADS) m = fmaxf(m, row[i] * inv_t);
    m = block_max(m, scratch);
    float s = 0.0f;
    for (int i = threadIdx.x; i < V; i += SAMPLE_THREADS) {
        const float e = expf(row[i] * inv_t - m);
        p[i] = e;
        s += e;
    }
    s = block_sum(s, scratch);
    {
        const float inv = 1.0f / s;
        for (int i = threadIdx.x; i < V; i += SAMPLE_THREADS) p[i] *= inv;
    }
    __syncthreads();

    // top-k: keep everything not below the k-th largest probability.
    const int k = top_k[r];
    if (k > 0 && k < V) {
        unsigned lo = 0u, hi = 0x7f800000u;
        while (lo < hi) {
            const unsigned mid = lo + (hi - lo + 1u) / 2u;
            float c = 0.0f;
            for (int i = threadIdx.x; i < V; i += SAMPLE_THREADS) c += (__float_as_uint(p[i]) >= mid) ? 1.0f : 0.0f;
            c = block_sum(c, scratch);
            if (c >= (float)k) lo = mid; else hi = mid - 1u;
        }
        const float kth = __uint_as_float(lo);
        for (int i = threadIdx.x; i < V; i += SAMPLE_THREADS) if (p[i] < kth) p[i] = 0.0f;
        __syncthreads();
        normalize_row(p, V, scratch);
    }

    // min-p: drop what is below min_p * the largest probability.
    const float mp = min_p[r];
    if (mp > 0.0f) {
        float mx = 0.0f;
        for (int i = threadIdx.x; i < V; i += SAMPLE_THREADS) mx = fmaxf(mx, p[i]);
        mx = block_max(mx, scratch);
        const float thr = mp * mx;
        for (int i = threadIdx.x; i < V; i += SAMPLE_THREADS) if (p[i] < thr) p[i] = 0.0f;
        __syncthreads();
    }

    // top-p: the smallest set of the most probable tokens whose mass reaches top_p; equal
    // probabilities at the cut stay together.
    const float tp = top_p[r];
    if (tp > 0.0f && tp < 1.0f) {
        unsigned lo = 0u, hi = 0x7f800000u;
        while (lo < hi) {
            const unsigned mid = lo + (hi - lo + 1u) / 2u;
            float mass = 0.0f;
            for (int i = threadIdx.x; i < V; i += SAMPLE_THREADS) mass += (__float_as_uint(p[i]) >= mid) ? p[i] : 0.0f;
            mass = block_sum(mass, scratch);
            if (mass >= tp) lo = mid; else hi = mid - 1u;
        }
        const float cut = __uint_as_float(lo);
        for (int i = threadIdx.x; i < V; i += SAMPLE_THREADS) if (p[i] < cut) p[i] = 0.0f;
        __syncthreads();
    }
    normalize_row(p, V, scratch);

    // inverse CDF: thread j owns the contiguous slice [j*chunk, (j+1)*chunk).
    const int chunk = (V + SAMPLE_THREADS - 1) / SAMPLE_THREADS;
    const int c0 = min(V, threadIdx.x * chunk), c1 = min(V, c0 + chunk);
    float part = 0.0f;
    for (int i = c0; i < c1; ++i) part += p[i];
    prefix_s[threadIdx.x] = part;
    if (threadIdx.x == 0) pick_s = 0x7fffffff;
    __syncthreads();
    if (threadIdx.x == 0) {  // serial inclusive scan: 1024 additions in a fixed order
        float run = 0.0f;
        for (int j = 0; j < SAMPLE_THREADS; ++j) {
            run += prefix_s[j];
            prefix_s[j] = run;
        }
    }
    __syncthreads();
    const float u = uniform[r];
    const float before = threadIdx.x == 0 ? 0.0f : prefix_s[threadIdx.x - 1];
    if (c1 > c0 && u <= prefix_s[threadIdx.x] && u > before) {
        float run = before;
        int pick = -1;
        for (int i = c0; i < c1; ++i) {
            run += p[i];
            if (u <= run && p[i] > 0.0f) {
                pick = i;
                break;
            }
        }
        if (pick < 0)  // rounding between the slice sum and the running sum: last kept token of the slice
            for (int i = c1 - 1; i >= c0; --i) if (p[i] > 0.0f) { pick = i; break; }
        if (pick >= 0) atomicMin(&pick_s, pick);
    }
    __syncthreads();
    if (pick_s == 0x7fffffff) {
        // u beyond the total mass (rounding): the last token that kept a probability.
        ArgBest mine;
        mine.v = -INFINITY;
        mine.i = 0x7fffffff;
        for (int i = threadIdx.x; i < V; i += SAMPLE_THREADS)
            if (p[i] > 0.0f) { mine.v = (float)i; mine.i = i; }
        ArgBest last = block_argmax(mine, ascratch);
        if (threadIdx.x == 0) out[r] = last.i == 0x7fffffff ? V - 1 : last.i;
    } else if (threadIdx.x == 0) {
        out[r] = pick_s;
    }
}

SHARPI_API int sharpi_sample_rows(const float* logits, int R, int V, const float* temperature, const int* top_k,
                                  const float* top_p, const float* min_p, const float* uniform, float* probs,
                                  int* out, cudaStream_t stream) {
    if (R <= 0) return SHARPI_OK;
    if (V <= 0 || V > (1 << 24)) return SHARPI_BAD_ARGUMENT;
    sample_rows_kernel<<<R, SAMPLE_THREADS, 0, stream>>>(logits, V, temperature, top_k, top_p, min_p, uniform,
                                                         probs, out);
    SHARPI_CHECK_LAUNCH();
    return SHARPI_OK;
}

// ---------------------------------------------------------------------------------------
// The same sampler for callers that cannot allocate device memory: the [rows, vocab] work area is
// a file-scope device array of this library.  See sampling_no_alloc.h for who needs it and for the
// rules (size limit, first call per device, shared contents, no overlapping calls).
// ---------------------------------------------------------------------------------------
#include <mutex>

#include "sampling_no_alloc.h"

static __device__ __align__(256) float g_no_alloc_probs[SHARPI_NO_ALLOC_MAX_FLOATS];

// In host code `g_no_alloc_probs` is only a handle for the runtime, not a device address: handing it
// to a kernel would make the kernel read host memory or fault.  The address the kernel needs comes
// from cudaGetSymbolAddress, asked once per device with that device current.
static float* no_alloc_work_area(int* status) {
    constexpr int MAX_DEVICES = 64;
    static float* per_device[MAX_DEVICES] = {};
    static std::mutex guard;
    int device = -1;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= MAX_DEVICES) {
        *status = SHARPI_NO_ALLOC_SETUP_FAILED;
        return nullptr;
    }
    std::lock_guard<std::mutex> hold(guard);
    if (per_device[device] == nullptr) {
        float* address = nullptr;
        if (cudaGetSymbolAddress((void**)&address, g_no_alloc_probs) != cudaSuccess || address == nullptr) {
            cudaGetLastError();  // leave no sticky error behind for the caller's next launch check
            *status = SHARPI_NO_ALLOC_SETUP_FAILED;
            return nullptr;
        }
        per_device[device] = address;
    }
    return per_device[device];
}

int sharpi_sample_rows_no_alloc(const float* logits, int rows, int vocab, const float* temperature,
                                const int* top_k, const float* top_p, const float* min_p, const float* uniform,
                                int* out, cudaStream_t stream) {
    if (rows <= 0) return SHARPI_OK;
    if (vocab <= 0 || vocab > (1 << 24)) return SHARPI_BAD_ARGUMENT;
    if ((unsigned long long)rows * (unsigned long long)vocab > (unsigned long long)SHARPI_NO_ALLOC_MAX_FLOATS)
        return SHARPI_NO_ALLOC_TOO_LARGE;
    int status = SHARPI_OK;
    float* probs = no_alloc_work_area(&status);
    if (probs == nullptr) return status;
    sample_rows_kernel<<<rows, SAMPLE_THREADS, 0, stream>>>(logits, vocab, temperature, top_k, top_p, min_p,
                                                            uniform, probs, out);
    SHARPI_CHECK_LAUNCH();
    return SHARPI_OK;
}
