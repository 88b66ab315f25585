// Temperature sampling with top-k / min-p / top-p for large vocabularies, every row cut over 32 blocks.
//
// The one-block-per-row sampler (sampling.cu) walks a row of 202048 logits some seventy times (two
// thirty-one-step searches for the top-k and top-p thresholds): 0.7 ms a step on one SM.  Here a row's
// work is spread over SLICES blocks and the thresholds are found by radix selection: three passes of
// histograms over the bits of the unnormalised probability e = exp(x / T - max) (11, 11 and 9 bits from
// the top), first by count for top-k, then by mass for top-p.  Probability mass is kept in fixed point
// (e * 2^40 in 64-bit integers), so every sum is exact, the order of the additions does not matter, and
// integer atomics give the same result in every run: a request's tokens do not depend on scheduling.
//
// The rules are those of sample_rows_kernel (src/SharpInference.Engine/Sampler.cs:71-107 in the
// reference: filters in the order top-k, min-p, top-p after the softmax):
//   top-k   keep everything not below the k-th largest probability (ties stay together)
//   min-p   drop what is below min_p times the largest probability (e = 1 at the largest)
//   top-p   the smallest set of the most probable tokens whose mass reaches top_p of what top-k kept;
//           equal probabilities at the cut stay together
//   draw    the first token, in the order of the vocabulary, at which the running mass of the kept
//           tokens exceeds u times their total
// Kernels of one call follow each other on the stream; between them the state of a row lives in
// `SampleRow`, and the histograms and counters are left at zero by the block that used them last.
#include "common.cuh"

constexpr int SLICES = 32;
constexpr int SL_THREADS = 256;
constexpr int BINS = 2048;
constexpr float MASS_SCALE = 1099511627776.0f;   // 2^40

struct SampleRow {
    float m;                          // largest x / T of the row
    int argmax;                       // its lowest index
    unsigned kth;                     // bits of the smallest e that top-k keeps (0: everything)
    unsigned cut;                     // bits of the smallest e that top-p keeps (0: everything)
    unsigned long long kept_mass;     // mass of what top-k keeps: what top_p is a fraction of
    unsigned prefix;                  // radix selection: the bits settled so far
    unsigned above_count;             // ... elements above the bin that is being refined
    unsigned long long above_mass;    // ... and their mass
    unsigned long long target;        // mass passes: the mass to reach
    int ticket;                       // blocks of the row that finished the running kernel
    int pad;
};

struct SlicedArgs {
    const float* logits;              // [R, V]
    const float* temperature;         // [R]; <= 0: the row takes its argmax
    const int* top_k;
    const float* top_p;
    const float* min_p;
    const float* uniform;
    SampleRow* rows;                  // [R]
    float* slice_max;                 // [R, SLICES]
    int* slice_arg;                   // [R, SLICES]
    unsigned* hist_count;             // [R, BINS] zero between kernels
    unsigned long long* hist_mass;    // [R, BINS] zero between kernels
    unsigned long long* slice_mass;   // [R, SLICES]
    int* out;                         // [R]
    int V;
};

__device__ __forceinline__ void slice_bounds(int V, int sl, int& begin, int& end) {
    const int per = (((V + SLICES - 1) / SLICES) + 3) & ~3;
    begin = min(V, sl * per);
    end = min(V, begin + per);
}

__device__ __forceinline__ float unnormalised(float x, float inv_t, float m) { return expf(x * inv_t - m); }

__device__ __forceinline__ unsigned long long fixed_mass(float e) { return (unsigned long long)(e * MASS_SCALE); }

// ---- kernel 1: the row's maximum and its index, slice by slice -------------------------------------
__global__ void __launch_bounds__(SL_THREADS) sliced_max_kernel(SlicedArgs a) {
    __shared__ float v_s[SL_THREADS / 32];
    __shared__ int i_s[SL_THREADS / 32];
    pdl_wait();
    const int r = blockIdx.y, sl = blockIdx.x;
    int begin, end;
    slice_bounds(a.V, sl, begin, end);
    const float* row = a.logits + (size_t)r * a.V;
    float best = -INFINITY;
    int arg = 0x7fffffff;
    for (int i = begin + threadIdx.x; i < end; i += SL_THREADS) {
        const float v = row[i];
        if (v > best) {          // ascending i per thread: strict > keeps the lowest index
            best = v;
            arg = i;
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, arg, o);
        if (ov > best || (ov == best && oi < arg)) {
            best = ov;
            arg = oi;
        }
    }
    if ((threadIdx.x & 31) == 0) {
        v_s[threadIdx.x >> 5] = best;
        i_s[threadIdx.x >> 5] = arg;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < SL_THREADS / 32; ++w)
            if (v_s[w] > best || (v_s[w] == best && i_s[w] < arg)) {
                best = v_s[w];
                arg = i_s[w];
            }
        a.slice_max[r * SLICES + sl] = best;
        a.slice_arg[r * SLICES + sl] = arg;
        if (sl == 0) {                  // thresholds of an earlier call must not outlive it
            a.rows[r].kth = 0;
            a.rows[r].cut = 0;
        }
    }
}

// The row's maximum from the slices' (every block of the later kernels forms it the same way).
__device__ __forceinline__ void row_max(const SlicedArgs& a, int r, float& best, int& arg) {
    best = -INFINITY;
    arg = 0x7fffffff;
    for (int s = 0; s < SLICES; ++s) {
        const float v = a.slice_max[r * SLICES + s];
        const int i = a.slice_arg[r * SLICES + s];
        if (v > best || (v == best && i < arg)) {
            best = v;
            arg = i;
        }
    }
}

// ---- kernels 2 .. 7: one pass of radix selection ---------------------------------------------------
// pass 0, 1, 2 take bits 30..20, 19..9, 8..0 of e's pattern.  by_mass = 0: towards the k-th largest
// (count); 1: towards the top-p cut (mass of the elements that top-k and min-p keep).

__global__ void __launch_bounds__(SL_THREADS) sliced_pass_kernel(SlicedArgs a, int pass, int by_mass) {
    __shared__ unsigned count_s[BINS];
    __shared__ unsigned long long mass_s[BINS];
    __shared__ unsigned long long part_mass_s[SL_THREADS];
    __shared__ unsigned part_count_s[SL_THREADS];
    __shared__ int last_s, found_s;
    pdl_wait();
    const int r = blockIdx.y, sl = blockIdx.x;
    const float temp = a.temperature[r];
    const int k = a.top_k[r];
    const float tp = a.top_p[r];
    const bool wants_k = k > 0 && k < a.V;
    const bool wants_p = tp > 0.0f && tp < 1.0f;
    SampleRow* st = a.rows + r;
    // rows that do not take part in this kind of pass leave at once (uniform over the row's blocks);
    // the first counting pass also runs for rows with top-p alone: it gives the row's whole mass
    if (temp <= 0.0f) return;
    if (by_mass ? !wants_p : (pass > 0 ? !wants_k : !(wants_k || wants_p))) return;

    const int shift = pass == 0 ? 20 : pass == 1 ? 9 : 0, bits = pass == 2 ? 9 : 11, bins = 1 << bits;
    for (int b = threadIdx.x; b < bins; b += SL_THREADS) {
        count_s[b] = 0;
        mass_s[b] = 0;
    }
    float mx;
    int arg;
    row_max(a, r, mx, arg);
    const float inv_t = 1.0f / temp, m = mx * inv_t;
    const unsigned prefix = pass == 0 ? 0u : st->prefix;          // settled bits, in place
    const unsigned settled_mask = pass == 0 ? 0u : (0x7fffffffu >> (shift + bits)) << (shift + bits);
    const unsigned floor_bits = by_mass ? max(st->kth, __float_as_uint(fmaxf(a.min_p[r], 0.0f))) : 0u;
    __syncthreads();
    int begin, end;
    slice_bounds(a.V, sl, begin, end);
    const float* row = a.logits + (size_t)r * a.V;
    for (int i = begin + threadIdx.x; i < end; i += SL_THREADS) {
        const float e = unnormalised(row[i], inv_t, m);
        const unsigned key = __float_as_uint(e);
        if ((key & settled_mask) != prefix) continue;
        if (key < floor_bits) continue;                             // not kept by top-k / min-p
        const unsigned b = (key >> shift) & (bins - 1);
        atomicAdd(&count_s[b], 1u);
        atomicAdd(&mass_s[b], fixed_mass(e));
    }
    __syncthreads();
    unsigned* hc = a.hist_count + (size_t)r * BINS;
    unsigned long long* hm = a.hist_mass + (size_t)r * BINS;
    for (int b = threadIdx.x; b < bins; b += SL_THREADS)
        if (count_s[b]) {
            atomicAdd(&hc[b], count_s[b]);
            atomicAdd(&hm[b], mass_s[b]);
        }
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        last_s = (atomicAdd(&st->ticket, 1) == SLICES - 1);
        if (last_s) st->ticket = 0;
        found_s = -1;
    }
    __syncthreads();
    if (!last_s) return;
    __threadfence();

    // The last block of the row walks the bins from the top: thread t owns the bins
    // [t * per_thread, (t + 1) * per_thread); it leaves the histograms at zero.
    const int per_thread = bins / SL_THREADS > 0 ? bins / SL_THREADS : 1;
    const int owners = bins / per_thread;
    unsigned my_count = 0;
    unsigned long long my_mass = 0;
    unsigned c[8];
    unsigned long long mm[8];
    if ((int)threadIdx.x < owners) {
        for (int j = 0; j < per_thread; ++j) {
            const int b = threadIdx.x * per_thread + j;
            c[j] = __ldcg(&hc[b]);
            mm[j] = __ldcg(&hm[b]);
            hc[b] = 0;
            hm[b] = 0;
            my_count += c[j];
            my_mass += mm[j];
        }
    }
    part_count_s[threadIdx.x] = my_count;
    part_mass_s[threadIdx.x] = my_mass;
    __syncthreads();
    // what lies above this thread's bins, inside this pass's histogram: a suffix sum over the threads,
    // first inside each warp, then over the warps' totals
    unsigned up_count = my_count;
    unsigned long long up_mass = my_mass;
    const int lane = threadIdx.x & 31, wrp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const unsigned oc = __shfl_down_sync(0xffffffffu, up_count, o);
        const unsigned long long om = __shfl_down_sync(0xffffffffu, up_mass, o);
        if (lane + o < 32) {
            up_count += oc;
            up_mass += om;
        }
    }
    __syncthreads();
    if (lane == 0) {                       // lane 0 holds its warp's total
        part_count_s[wrp] = up_count;
        part_mass_s[wrp] = up_mass;
    }
    __syncthreads();
    unsigned long long all_mass = 0;       // the whole histogram's mass (the row's mass in the first counting pass)
    for (int w = 0; w < SL_THREADS / 32; ++w) all_mass += part_mass_s[w];
    for (int w = wrp + 1; w < SL_THREADS / 32; ++w) {
        up_count += part_count_s[w];
        up_mass += part_mass_s[w];
    }
    up_count -= my_count;                  // strictly above this thread's bins
    up_mass -= my_mass;
    const unsigned base_count = pass == 0 ? 0u : st->above_count;
    const unsigned long long base_mass = pass == 0 ? 0ull : st->above_mass;
    unsigned long long target = 0;
    if (by_mass) {
        if (pass == 0) {
            const double want = (double)tp * (double)st->kept_mass;
            target = (unsigned long long)want;
            if (target < 1) target = 1;
        } else {
            target = st->target;
        }
    }
    __syncthreads();
    // exactly one thread's range holds the crossing (or none: then the lowest bin is taken)
    if ((int)threadIdx.x < owners) {
        const bool below = by_mass ? base_mass + up_mass < target : base_count + up_count < (unsigned)k;
        const bool reach = by_mass ? base_mass + up_mass + my_mass >= target
                                   : base_count + up_count + my_count >= (unsigned)k;
        if (below && reach) found_s = threadIdx.x;
    }
    __syncthreads();
    // the first counting pass always leaves the row's whole mass (rows without top-k: what top-p refers to)
    if (!by_mass && pass == 0 && threadIdx.x == 0 && !wants_k) {
        st->kept_mass = all_mass;
        st->kth = 0;
    }
    if (!by_mass && !wants_k) return;
    const int owner = found_s < 0 ? 0 : found_s;
    if ((int)threadIdx.x != owner) return;
    unsigned cc = base_count + up_count;
    unsigned long long cm = base_mass + up_mass;
    int pick = threadIdx.x * per_thread;                  // the lowest bin of the range, if nothing crosses
    for (int j = per_thread - 1; j >= 0; --j) {
        const bool reach = by_mass ? cm + mm[j] >= target : cc + c[j] >= (unsigned)k;
        if (reach || j == 0) {          // j == 0 without reach: nothing crosses, the lowest bin keeps everything
            pick = threadIdx.x * per_thread + j;
            const unsigned new_prefix = prefix | ((unsigned)pick << shift);
            if (pass == 2) {
                if (by_mass) {
                    st->cut = new_prefix;
                } else {
                    st->kth = new_prefix;
                    st->kept_mass = cm + mm[j];           // everything not below the k-th largest
                }
            } else {
                st->prefix = new_prefix;
                st->above_count = cc;                     // what lies strictly above the picked bin
                st->above_mass = cm;
                if (by_mass) st->target = target;
            }
            break;
        }
        cc += c[j];
        cm += mm[j];
    }
}

// ---- kernel 8: draw ---------------------------------------------------------------------------------
__global__ void __launch_bounds__(SL_THREADS) sliced_draw_kernel(SlicedArgs a) {
    __shared__ unsigned long long part_s[SL_THREADS];
    __shared__ unsigned long long slice_s[SLICES];
    __shared__ int last_s, pick_s;
    pdl_wait();
    const int r = blockIdx.y, sl = blockIdx.x;
    SampleRow* st = a.rows + r;
    const float temp = a.temperature[r];
    float mx;
    int arg;
    row_max(a, r, mx, arg);
    if (temp <= 0.0f) {
        if (sl == 0 && threadIdx.x == 0) a.out[r] = arg == 0x7fffffff ? 0 : arg;
        return;
    }
    const float inv_t = 1.0f / temp, m = mx * inv_t;
    const unsigned floor_bits = max(max(st->kth, st->cut), __float_as_uint(fmaxf(a.min_p[r], 0.0f)));
    const float* row = a.logits + (size_t)r * a.V;
    int begin, end;
    slice_bounds(a.V, sl, begin, end);
    unsigned long long mine = 0;
    for (int i = begin + threadIdx.x; i < end; i += SL_THREADS) {
        const float e = unnormalised(row[i], inv_t, m);
        if (__float_as_uint(e) >= floor_bits) mine += fixed_mass(e);
    }
    part_s[threadIdx.x] = mine;
    __syncthreads();
    if (threadIdx.x == 0) {
        unsigned long long total = 0;
        for (int t = 0; t < SL_THREADS; ++t) total += part_s[t];
        a.slice_mass[r * SLICES + sl] = total;
        __threadfence();
        last_s = (atomicAdd(&st->ticket, 1) == SLICES - 1);
        if (last_s) st->ticket = 0;
    }
    __syncthreads();
    if (!last_s) return;
    __threadfence();
    // the row's last block: which slice holds the target, then which element of it
    if (threadIdx.x < SLICES) slice_s[threadIdx.x] = __ldcg(&a.slice_mass[r * SLICES + threadIdx.x]);
    __syncthreads();
    unsigned long long total = 0;
    for (int s = 0; s < SLICES; ++s) total += slice_s[s];
    if (total == 0) {                                    // nothing kept a mass (cannot happen: e = 1 at the maximum)
        if (threadIdx.x == 0) a.out[r] = arg == 0x7fffffff ? 0 : arg;
        return;
    }
    unsigned long long target = (unsigned long long)((double)a.uniform[r] * (double)total);
    if (target >= total) target = total - 1;
    int hit = 0;
    unsigned long long before = 0;
    for (int s = 0; s < SLICES; ++s) {
        if (target < before + slice_s[s]) {
            hit = s;
            break;
        }
        before += slice_s[s];
    }
    // inside the slice: thread t owns a contiguous run of elements
    slice_bounds(a.V, hit, begin, end);
    const int n = end - begin, chunk = (n + SL_THREADS - 1) / SL_THREADS;
    const int c0 = begin + min(n, (int)threadIdx.x * chunk), c1 = begin + min(n, (int)(threadIdx.x + 1) * chunk);
    unsigned long long run = 0;
    for (int i = c0; i < c1; ++i) {
        const float e = unnormalised(row[i], inv_t, m);
        if (__float_as_uint(e) >= floor_bits) run += fixed_mass(e);
    }
    __syncthreads();
    part_s[threadIdx.x] = run;
    if (threadIdx.x == 0) pick_s = -1;
    __syncthreads();
    unsigned long long lower = before;
    for (int t = 0; t < (int)threadIdx.x; ++t) lower += part_s[t];
    if (target >= lower && target < lower + run) {       // exactly one thread
        unsigned long long acc = lower;
        for (int i = c0; i < c1; ++i) {
            const float e = unnormalised(row[i], inv_t, m);
            if (__float_as_uint(e) >= floor_bits) {
                acc += fixed_mass(e);
                if (target < acc) {
                    pick_s = i;
                    break;
                }
            }
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) a.out[r] = pick_s >= 0 ? pick_s : (arg == 0x7fffffff ? 0 : arg);
}

// `work`: scratch that is all zero before the first call and is left so by every call (its size:
// sharpi_sample_rows_sliced_work_bytes(R)).  `any_top_k` / `any_top_p`: whether any row uses the filter
// (the passes of a filter that no row uses are not launched).
SHARPI_API long long sharpi_sample_rows_sliced_work_bytes(int R) {
    if (R <= 0) return 0;
    return (long long)R * (sizeof(SampleRow) + SLICES * (sizeof(float) + sizeof(int) + sizeof(unsigned long long)) +
                           BINS * (sizeof(unsigned) + sizeof(unsigned long long))) + 256;
}

SHARPI_API int sharpi_sample_rows_sliced(const float* logits, int R, int V, const float* temperature, const int* top_k,
                                         const float* top_p, const float* min_p, const float* uniform, void* work,
                                         int any_top_k, int any_top_p, int* out, cudaStream_t stream) {
    if (R <= 0) return SHARPI_OK;
    if (V <= 0 || V > (1 << 24) || R > 65535 || !work) return SHARPI_BAD_ARGUMENT;
    if (reinterpret_cast<uintptr_t>(work) & 15) return SHARPI_UNALIGNED;
    SlicedArgs a;
    a.logits = logits; a.temperature = temperature; a.top_k = top_k; a.top_p = top_p; a.min_p = min_p;
    a.uniform = uniform; a.out = out; a.V = V;
    char* p = reinterpret_cast<char*>(work);
    a.rows = reinterpret_cast<SampleRow*>(p);               p += (size_t)R * sizeof(SampleRow);
    a.hist_mass = reinterpret_cast<unsigned long long*>(p); p += (size_t)R * BINS * sizeof(unsigned long long);
    a.slice_mass = reinterpret_cast<unsigned long long*>(p); p += (size_t)R * SLICES * sizeof(unsigned long long);
    a.hist_count = reinterpret_cast<unsigned*>(p);          p += (size_t)R * BINS * sizeof(unsigned);
    a.slice_max = reinterpret_cast<float*>(p);              p += (size_t)R * SLICES * sizeof(float);
    a.slice_arg = reinterpret_cast<int*>(p);
    const dim3 grid(SLICES, R);
    SHARPI_LAUNCH_PDL(sliced_max_kernel, grid, SL_THREADS, 0, stream, a);
    if (any_top_k || any_top_p) SHARPI_LAUNCH_PDL(sliced_pass_kernel, grid, SL_THREADS, 0, stream, a, 0, 0);
    if (any_top_k) {
        SHARPI_LAUNCH_PDL(sliced_pass_kernel, grid, SL_THREADS, 0, stream, a, 1, 0);
        SHARPI_LAUNCH_PDL(sliced_pass_kernel, grid, SL_THREADS, 0, stream, a, 2, 0);
    }
    if (any_top_p) {
        SHARPI_LAUNCH_PDL(sliced_pass_kernel, grid, SL_THREADS, 0, stream, a, 0, 1);
        SHARPI_LAUNCH_PDL(sliced_pass_kernel, grid, SL_THREADS, 0, stream, a, 1, 1);
        SHARPI_LAUNCH_PDL(sliced_pass_kernel, grid, SL_THREADS, 0, stream, a, 2, 1);
    }
    SHARPI_LAUNCH_PDL(sliced_draw_kernel, grid, SL_THREADS, 0, stream, a);
    return SHARPI_OK;
}
