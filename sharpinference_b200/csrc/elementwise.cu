// Embedding lookup, residual-add + RMSNorm, SwiGLU and dtype casts.
//
// The residual stream is fp32 in both precisions; sums of squares, the rsqrt and the
// scaling are fp32.  Counterparts in the reference: llm_embed_lookup_f32
// (src/SharpInference.Cuda/CudaTextKernels.cs:944), llm_rmsnorm / llm_rmsnorm_batched
// (:199, :5819), add_inplace (src/SharpInference.Cuda/CudaKernels.cs:89) and llm_silu_mul
// (CudaTextKernels.cs:331); here the residual add is fused into the norm that follows it.
#include "common.cuh"

// ---------------------------------------------------------------------------------------
// out[t, :] = table[ids[t], :]           (fp32 residual stream)
// ---------------------------------------------------------------------------------------
template <typename TT>
__global__ void embed_gather_kernel(const int* __restrict__ ids, const TT* __restrict__ table,
                                    float* __restrict__ out, int H, int V) {
    const int t = blockIdx.x;
    int id = ids[t];
    const bool valid = (id >= 0 && id < V);
    const TT* row = table + (size_t)(valid ? id : 0) * H;
    float* dst = out + (size_t)t * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) dst[i] = valid ? to_float(row[i]) : 0.0f;
}

SHARPI_API int sharpi_embed_gather(const int* ids, const void* table, int table_dtype, float* out,
                                   int T, int H, int V, cudaStream_t stream) {
    if (T <= 0) return SHARPI_OK;
    if (H <= 0 || V <= 0) return SHARPI_BAD_ARGUMENT;
    const int threads = H >= 1024 ? 256 : 128;
    if (table_dtype == SHARPI_F32)
        embed_gather_kernel<float><<<T, threads, 0, stream>>>(ids, (const float*)table, out, H, V);
    else if (table_dtype == SHARPI_BF16)
        embed_gather_kernel<bf16><<<T, threads, 0, stream>>>(ids, (const bf16*)table, out, H, V);
    else
        return SHARPI_BAD_ARGUMENT;
    SHARPI_CHECK_LAUNCH();
    return SHARPI_OK;
}

// ---------------------------------------------------------------------------------------
// Residual add + RMSNorm.
//   rows == nullptr:  x[t] += delta[t] (written back); out[t] = x[t] * rsqrt(mean(x[t]^2)+eps) * w
//                     (w == nullptr: the weightless norm, src/SharpInference.Cpu/SimdKernels.cs:4252-4283)
//   rows != nullptr:  r = rows[t]; v = x[r] + delta[r] (x untouched); out[t] = norm(v)
// `out` has dtype out_dtype; `out32` (optional) receives the same values in fp32, for
// consumers that must not see them rounded (the expert router).
// One block of NORM_THREADS threads per row whatever the batch, so the order of the
// additions in the sum of squares never depends on what else is in the step.
// ---------------------------------------------------------------------------------------
constexpr int NORM_THREADS = 256;

// The row is read in pieces of NORM_UNROLL elements per thread whose loads are all issued before the first
// of them is used (a step of few rows is one block per row waiting for memory, nothing else), and kept in
// shared memory for the second pass when it fits (CACHED).  A thread still adds its squares in ascending
// order of the index, as a plain loop would.
constexpr int NORM_UNROLL = 8;
constexpr int NORM_CACHE_FLOATS = 12288;     // 48 KB

// WIDE_ORDER: the sum of squares is formed in the order of add_rmsnorm_wide_kernel below (as if 1024 threads each
// added their own elements and the block's tree were that of 32 warps), so that a row gives the same bits
// whichever of the two kernels a step of its size takes: this thread stands for the virtual threads
// t, t + 256, t + 512, t + 768.
template <typename TO, bool CACHED, bool WIDE_ORDER>
__global__ void __launch_bounds__(NORM_THREADS)
add_rmsnorm_kernel(float* x, const float* __restrict__ delta, const float* __restrict__ w, float eps,
                   const int* __restrict__ rows, int H, TO* __restrict__ out, float* __restrict__ out32) {
    __shared__ float scratch[32];
    extern __shared__ float row_s[];
    pdl_wait();
    const int t = blockIdx.x;
    const size_t src = (size_t)(rows ? rows[t] : t) * H;
    float* xr = x + src;
    const float* dr = delta ? delta + src : nullptr;
    const bool write_back = dr && !rows;
    float ss = 0.0f;
    float ss4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    for (int i0 = threadIdx.x; i0 < H; i0 += NORM_UNROLL * NORM_THREADS) {
        float v[NORM_UNROLL], d[NORM_UNROLL];
#pragma unroll
        for (int k = 0; k < NORM_UNROLL; ++k) {
            const int i = i0 + k * NORM_THREADS;
            v[k] = (i < H) ? xr[i] : 0.0f;
            d[k] = (dr && i < H) ? dr[i] : 0.0f;
        }
#pragma unroll
        for (int k = 0; k < NORM_UNROLL; ++k) {
            const int i = i0 + k * NORM_THREADS;
            if (i < H) {
                if (dr) v[k] += d[k];
                if (write_back) xr[i] = v[k];
                if (CACHED) row_s[i] = v[k];
                if (WIDE_ORDER) ss4[k & 3] += v[k] * v[k];
                else ss += v[k] * v[k];
            }
        }
    }
    if (WIDE_ORDER) {
        const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
        for (int a = 0; a < 4; ++a) ss4[a] = warp_sum(ss4[a]);
        __syncthreads();
        if (lane == 0) {
#pragma unroll
            for (int a = 0; a < 4; ++a) scratch[warp + (NORM_THREADS / 32) * a] = ss4[a];   // virtual warp w + 8 a
        }
        __syncthreads();
        ss = warp_sum(scratch[lane]);
    } else {
        ss = block_sum(ss, scratch);
    }
    const float scale = 1.0f / sqrtf(ss / (float)H + eps);
    TO* orow = out + (size_t)t * H;
    float* o32 = out32 ? out32 + (size_t)t * H : nullptr;
    for (int i0 = threadIdx.x; i0 < H; i0 += NORM_UNROLL * NORM_THREADS) {
        float v[NORM_UNROLL], ww[NORM_UNROLL];
#pragma unroll
        for (int k = 0; k < NORM_UNROLL; ++k) {
            const int i = i0 + k * NORM_THREADS;
            ww[k] = (i < H) ? (w ? w[i] : 1.0f) : 0.0f;
            if (CACHED) {
                v[k] = (i < H) ? row_s[i] : 0.0f;      // this thread wrote it
            } else {
                v[k] = (i < H) ? xr[i] : 0.0f;
                if (dr && rows && i < H) v[k] += dr[i];
            }
        }
#pragma unroll
        for (int k = 0; k < NORM_UNROLL; ++k) {
            const int i = i0 + k * NORM_THREADS;
            if (i < H) {
                const float y = v[k] * scale * ww[k];
                orow[i] = from_float<TO>(y);
                if (o32) o32[i] = y;
            }
        }
    }
}

// Rows of up to NORM_WIDE_THREADS * NORM_UNROLL elements: 1024 threads hold the whole row in registers, so every
// load of the row, of the update and of the weight is issued before anything is used and the kernel is two trips to
// memory long (a decode step runs this kernel two or three times a layer with one block per row: its latency, not
// its bandwidth, is what counts there).  A thread adds its squares in ascending order of the index; the block's
// tree is fixed by the block size, so a row's result does not depend on the batch.
constexpr int NORM_WIDE_THREADS = 1024;
constexpr int NORM_WIDE_ROWS = 128;       // steps of up to this many rows take it

template <typename TO>
__global__ void __launch_bounds__(NORM_WIDE_THREADS)
add_rmsnorm_wide_kernel(float* x, const float* __restrict__ delta, const float* __restrict__ w, float eps,
                        const int* __restrict__ rows, int H, TO* __restrict__ out, float* __restrict__ out32) {
    __shared__ float scratch[32];
    // the weight is written by no kernel: it may be on its way before the kernel ahead has finished
    float ww[NORM_UNROLL];
#pragma unroll
    for (int k = 0; k < NORM_UNROLL; ++k) {
        const int i = threadIdx.x + k * NORM_WIDE_THREADS;
        ww[k] = (i < H) ? (w ? w[i] : 1.0f) : 0.0f;
    }
    pdl_wait();
    const int t = blockIdx.x;
    const size_t src = (size_t)(rows ? rows[t] : t) * H;
    float* xr = x + src;
    const float* dr = delta ? delta + src : nullptr;
    const bool write_back = dr && !rows;
    float v[NORM_UNROLL], d[NORM_UNROLL];
#pragma unroll
    for (int k = 0; k < NORM_UNROLL; ++k) {
        const int i = threadIdx.x + k * NORM_WIDE_THREADS;
        v[k] = (i < H) ? xr[i] : 0.0f;
        d[k] = (dr && i < H) ? dr[i] : 0.0f;
    }
    float ss = 0.0f;
#pragma unroll
    for (int k = 0; k < NORM_UNROLL; ++k) {
        const int i = threadIdx.x + k * NORM_WIDE_THREADS;
        if (i < H) {
            if (dr) v[k] += d[k];
            if (write_back) xr[i] = v[k];
            ss += v[k] * v[k];
        }
    }
    ss = block_sum(ss, scratch);
    const float scale = 1.0f / sqrtf(ss / (float)H + eps);
    TO* orow = out + (size_t)t * H;
    float* o32 = out32 ? out32 + (size_t)t * H : nullptr;
#pragma unroll
    for (int k = 0; k < NORM_UNROLL; ++k) {
        const int i = threadIdx.x + k * NORM_WIDE_THREADS;
        if (i < H) {
            const float y = v[k] * scale * ww[k];
            orow[i] = from_float<TO>(y);
            if (o32) o32[i] = y;
        }
    }
}

template <typename TO>
static int launch_norm(float* x, const float* delta, const float* w, float eps, const int* rows, int T, int H, TO* out,
                       float* out32, cudaStream_t stream) {
    if (H <= NORM_WIDE_THREADS * NORM_UNROLL) {
        // few rows: latency counts (2.9 against 3.8 us at one row of 5120); many rows: bandwidth (33 against 49 us at
        // 2048 rows); the two kernels add in the same order, so the choice does not show in the result
        if (T <= NORM_WIDE_ROWS) {
            auto kern = add_rmsnorm_wide_kernel<TO>;
            SHARPI_LAUNCH_PDL(kern, T, NORM_WIDE_THREADS, 0, stream, x, delta, w, eps, rows, H, out, out32);
        } else {
            auto kern = add_rmsnorm_kernel<TO, true, true>;
            SHARPI_LAUNCH_PDL(kern, T, NORM_THREADS, (size_t)H * sizeof(float), stream, x, delta, w, eps, rows, H, out, out32);
        }
        return SHARPI_OK;
    }
    if (H <= NORM_CACHE_FLOATS) {
        auto kern = add_rmsnorm_kernel<TO, true, false>;
        SHARPI_LAUNCH_PDL(kern, T, NORM_THREADS, (size_t)H * sizeof(float), stream, x, delta, w, eps, rows, H, out, out32);
    } else {
        auto kern = add_rmsnorm_kernel<TO, false, false>;
        SHARPI_LAUNCH_PDL(kern, T, NORM_THREADS, 0, stream, x, delta, w, eps, rows, H, out, out32);
    }
    return SHARPI_OK;
}

SHARPI_API int sharpi_add_rmsnorm(float* x, const float* delta, const float* w, float eps, const int* rows,
                                  int T, int H, void* out, int out_dtype, float* out32, cudaStream_t stream) {
    if (T <= 0) return SHARPI_OK;
    if (H <= 0) return SHARPI_BAD_ARGUMENT;
    if (out_dtype == SHARPI_F32) return launch_norm<float>(x, delta, w, eps, rows, T, H, (float*)out, out32, stream);
    if (out_dtype == SHARPI_BF16) return launch_norm<bf16>(x, delta, w, eps, rows, T, H, (bf16*)out, out32, stream);
    return SHARPI_BAD_ARGUMENT;
}

// ---------------------------------------------------------------------------------------
// SwiGLU over a fused [M, 2I] gate|up product:  out[m, i] = silu(s*g) * (s*u),
// g = gate_up[m, i], u = gate_up[m, I + i], s = row_scale[scale_rows ? scale_rows[m] : m] or 1.
// The routed expert's router weight multiplies gate and up BEFORE the nonlinearity, which
// equals scaling the expert's input (src/SharpInference.Engine/ForwardPass.cs:2082-2088).
// ---------------------------------------------------------------------------------------
template <typename TO>
__global__ void swiglu_kernel(const float* __restrict__ gate_up, const float* __restrict__ row_scale,
                              const int* __restrict__ scale_rows, TO* __restrict__ out, int I) {
    const int m = blockIdx.x;
    const int i = blockIdx.y * blockDim.x + threadIdx.x;
    if (i >= I) return;
    const float s = row_scale ? row_scale[scale_rows ? scale_rows[m] : m] : 1.0f;
    const float g = gate_up[(size_t)m * 2 * I + i] * s;
    const float u = gate_up[(size_t)m * 2 * I + I + i] * s;
    const float act = g / (1.0f + expf(-g));
    out[(size_t)m * I + i] = from_float<TO>(act * u);
}

// Four elements per thread with 16-byte loads, for widths that are multiples of 4.
template <typename TO>
__global__ void swiglu_vec4_kernel(const float* __restrict__ gate_up, const float* __restrict__ row_scale,
                                   const int* __restrict__ scale_rows, TO* __restrict__ out, int I) {
    pdl_wait();
    const int m = blockIdx.x;
    const int i = (blockIdx.y * blockDim.x + threadIdx.x) * 4;
    if (i >= I) return;
    const float s = row_scale ? row_scale[scale_rows ? scale_rows[m] : m] : 1.0f;
    const float4 g4 = *reinterpret_cast<const float4*>(gate_up + (size_t)m * 2 * I + i);
    const float4 u4 = *reinterpret_cast<const float4*>(gate_up + (size_t)m * 2 * I + I + i);
    const float g[4] = {g4.x * s, g4.y * s, g4.z * s, g4.w * s};
    const float u[4] = {u4.x * s, u4.y * s, u4.z * s, u4.w * s};
    TO* dst = out + (size_t)m * I + i;
#pragma unroll
    for (int j = 0; j < 4; ++j) dst[j] = from_float<TO>(g[j] / (1.0f + expf(-g[j])) * u[j]);
}

SHARPI_API int sharpi_swiglu(const float* gate_up, const float* row_scale, const int* scale_rows, void* out,
                             int out_dtype, int M, int I, cudaStream_t stream) {
    if (M <= 0) return SHARPI_OK;
    if (I <= 0 || (I + 255) / 256 > 65535) return SHARPI_BAD_ARGUMENT;
    if (I % 4 == 0 && (reinterpret_cast<uintptr_t>(gate_up) & 15) == 0) {
        dim3 grid4(M, (I / 4 + 255) / 256);
        if (out_dtype == SHARPI_F32)
            SHARPI_LAUNCH_PDL(swiglu_vec4_kernel<float>, grid4, 256, 0, stream, gate_up, row_scale, scale_rows, (float*)out, I);
        else if (out_dtype == SHARPI_BF16)
            SHARPI_LAUNCH_PDL(swiglu_vec4_kernel<bf16>, grid4, 256, 0, stream, gate_up, row_scale, scale_rows, (bf16*)out, I);
        else
            return SHARPI_BAD_ARGUMENT;
        SHARPI_CHECK_LAUNCH();
        return SHARPI_OK;
    }
    dim3 grid(M, (I + 255) / 256);
    if (out_dtype == SHARPI_F32)
        swiglu_kernel<float><<<grid, 256, 0, stream>>>(gate_up, row_scale, scale_rows, (float*)out, I);
    else if (out_dtype == SHARPI_BF16)
        swiglu_kernel<bf16><<<grid, 256, 0, stream>>>(gate_up, row_scale, scale_rows, (bf16*)out, I);
    else
        return SHARPI_BAD_ARGUMENT;
    SHARPI_CHECK_LAUNCH();
    return SHARPI_OK;
}

// ---------------------------------------------------------------------------------------
// y[i] = a[i] + b[i] (fp32), used to combine a shared and a routed feed-forward output
// where no fused epilogue does it.
// ---------------------------------------------------------------------------------------
__global__ void add_kernel(const float* __restrict__ a, const float* __restrict__ b, float* __restrict__ y,
                           size_t n) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; i < n; i += stride) y[i] = a[i] + b[i];
}

SHARPI_API int sharpi_add(const float* a, const float* b, float* y, long long n, cudaStream_t stream) {
    if (n <= 0) return SHARPI_OK;
    long long blocks = (n + 255) / 256;
    if (blocks > 148 * 32) blocks = 148 * 32;
    add_kernel<<<(int)blocks, 256, 0, stream>>>(a, b, y, (size_t)n);
    SHARPI_CHECK_LAUNCH();
    return SHARPI_OK;
}

// y[m, n] += bias[n]: the bias of a projection whose product came from the library.
__global__ void add_bias_kernel(float* __restrict__ y, const float* __restrict__ bias, int N) {
    pdl_wait();
    const int n = blockIdx.y * blockDim.x + threadIdx.x;
    if (n < N) y[(size_t)blockIdx.x * N + n] += bias[n];
}

SHARPI_API int sharpi_add_bias(float* y, const float* bias, int M, int N, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return SHARPI_OK;
    if ((N + 255) / 256 > 65535) return SHARPI_BAD_ARGUMENT;
    dim3 grid(M, (N + 255) / 256);
    SHARPI_LAUNCH_PDL(add_bias_kernel, grid, 256, 0, stream, y, bias, N);
    return SHARPI_OK;
}

// The GPU's nanosecond clock into slot[index]: a marker between the launches of a stream, for timelines of a
// step taken inside a captured graph, where host-side timing sees nothing.
__global__ void timestamp_kernel(unsigned long long* slots, int index) {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    slots[index] = t;
}

SHARPI_API int sharpi_timestamp(unsigned long long* slots, int index, cudaStream_t stream) {
    if (!slots || index < 0) return SHARPI_BAD_ARGUMENT;
    timestamp_kernel<<<1, 1, 0, stream>>>(slots, index);
    SHARPI_CHECK_LAUNCH();
    return SHARPI_OK;
}
