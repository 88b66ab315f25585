// Dense products of a few rows (decode): out[m, n] = sum_k A[m, k] * W[n, k] for up to 16 rows of bfloat16
// activations against a bfloat16 weight [N, K] that is read exactly once.
//
// The product is bound by how fast the weight streams in, so the kernel is laid out for that alone:
//  * the weight rows are dealt out evenly over a grid of two CTAs per SM (each gets N / grid rows, one more or
//    less), every CTA takes its rows over the whole of K, so no partial sums cross CTAs, all SMs pull the same
//    share, and every output element is one sum in one fixed order whatever else is in the batch;
//  * a CTA walks its rows in groups of up to 32 (four tiles of eight rows: the n of mma m16n8k16); its eight
//    warps take every eighth 32-element piece of K; a lane loads 16 bytes of its weight row straight into
//    registers (no shared memory, nothing allocated in L1) and the matching 16 bytes of its activation row
//    through L1, where the few rows of activations stay for the CTAs of the SM; the activation registers serve
//    all four tiles, and several weight loads per lane are in flight before the first is used;
//  * the multiply-adds are mma.sync m16n8k16 (activations as the 16-row operand, weights as the 8-column one):
//    with so few rows the tensor cores are idle either way, and mma.sync takes its operands from registers,
//    which is where the loads put them.  The K positions inside a 32-element piece are dealt to the lanes in
//    16-byte runs (lane t of a row holds elements 8t .. 8t+7), the same for both operands, so the sum is over
//    the same products as with the standard fragment order;
//  * the first weight loads are issued before the kernel waits for the kernel before it: weights are written by
//    nobody, so where the kernel is started early (programmatic dependent launch) the stream begins during the
//    predecessor's tail (the host launches it the plain way, see launch_variant);
//  * the warps' partial sums meet in shared memory and are added in warp order; the epilogue stores (with an
//    optional bias), adds into the output with reductions (one addend per element from this launch), or applies
//    SwiGLU (a tile of gate rows and the tile of their up rows side by side) and writes bfloat16.
//
// The reference runs its single-token products on matvec kernels of its own and takes a library only for
// batched projections (src/SharpInference.Cuda/CudaTextKernels.cs:1325 llm_matvec_f32,
// src/SharpInference.Cuda/CudaBackend.cs:2083-2117).
#include "common.cuh"

namespace {

constexpr int DR_WARPS = 8;
constexpr int DR_THREADS = DR_WARPS * 32;
constexpr int DR_TILE = 8;          // weight rows per tile (the n of m16n8k16)
constexpr int DR_CTAS_PER_SM = 2;

enum DenseRowsMode : int { DR_STORE = 0, DR_ADD = 1, DR_SWIGLU = 2 };

__device__ __forceinline__ uint4 load_stream(const uint4* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

// Activations are the output of the kernel before this one, and where this kernel is started early it is running
// before that one has ended: they are read with an ordinary load that stays behind the wait (a load marked as
// reading memory that never changes, as __ldg is, may be moved ahead of it by the compiler: it was, and read the
// last step's values).
__device__ __forceinline__ uint4 load_after_wait(const uint4* p) {
    uint4 v;
    asm volatile("ld.global.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p)
                 : "memory");
    return v;
}

__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
        "{%0, %1, %2, %3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

struct DenseRowsParams {
    const bf16* A;          // [M, K]
    const bf16* W;          // [N, K]
    const float* bias;      // [N] or null (DR_STORE)
    void* out;              // fp32 [M, N], or bf16 [M, N / 2] with DR_SWIGLU
    int M, N, K;
};

// WIDE: more than eight activation rows.  DR_TILES: tiles of eight weight rows per group (with SwiGLU half of them
// gate rows, half their up rows); DR_U: adjacent 32-element pieces of K per step of a warp, so a lane's loads of
// a step cover DR_U * 64 bytes of its row in a run.  DR_TILES * DR_U 16-byte loads per lane are in flight.
template <int MODE, bool WIDE, int DR_TILES, int DR_U>
__global__ void __launch_bounds__(DR_THREADS, DR_CTAS_PER_SM)
dense_rows_kernel(const DenseRowsParams p) {
    static_assert(MODE != DR_SWIGLU || DR_TILES % 2 == 0, "gate and up tiles come in pairs");
    constexpr int ROWS = WIDE ? 16 : 8;
    // output rows of W a group covers: with SwiGLU tiles 0, 1 hold gate rows and tiles 2, 3 their up rows
    constexpr int GROUP = MODE == DR_SWIGLU ? DR_TILES / 2 * DR_TILE : DR_TILES * DR_TILE;
    __shared__ float part[DR_WARPS][DR_TILES][ROWS][DR_TILE];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int n_out = MODE == DR_SWIGLU ? p.N / 2 : p.N;
    // this CTA's output rows
    const int r_begin = (int)((long long)n_out * blockIdx.x / gridDim.x);
    const int r_end = (int)((long long)n_out * (blockIdx.x + 1) / gridDim.x);
    const int pieces = p.K >> 3;                        // 16-byte pieces of a row
    const int steps = (pieces + 4 * DR_U - 1) / (4 * DR_U);   // runs of DR_U * 32 elements of K
    const uint4* a_lo = reinterpret_cast<const uint4*>(p.A + (size_t)min(g, p.M - 1) * p.K);
    const uint4* a_hi = WIDE ? reinterpret_cast<const uint4*>(p.A + (size_t)min(g + 8, p.M - 1) * p.K) : nullptr;
    const bool lo_ok = g < p.M, hi_ok = WIDE && g + 8 < p.M;
    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
    bool waited = false;

    for (int r0 = r_begin; r0 < r_end; r0 += GROUP) {
        const uint4* wrow[DR_TILES];
        bool row_ok[DR_TILES];
#pragma unroll
        for (int i = 0; i < DR_TILES; ++i) {
            // output row of this lane in tile i, and the weight row it reads
            const int r = MODE == DR_SWIGLU ? r0 + (i % (DR_TILES / 2)) * DR_TILE + g : r0 + i * DR_TILE + g;
            row_ok[i] = r < r_end;
            const int wr = min(r, r_end - 1) + (MODE == DR_SWIGLU && i >= DR_TILES / 2 ? n_out : 0);
            wrow[i] = reinterpret_cast<const uint4*>(p.W + (size_t)wr * p.K);
        }
        float c[DR_TILES][4];
#pragma unroll
        for (int i = 0; i < DR_TILES; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) c[i][j] = 0.0f;

        for (int s = warp; s < steps; s += DR_WARPS) {
            uint4 wv[DR_TILES][DR_U], av[WIDE ? 2 : 1][DR_U];
#pragma unroll
            for (int u = 0; u < DR_U; ++u) {
                const int piece = (s * DR_U + u) * 4 + t;
#pragma unroll
                for (int i = 0; i < DR_TILES; ++i)
                    wv[i][u] = (piece < pieces && row_ok[i]) ? load_stream(wrow[i] + piece) : zero;
            }
            if (!waited) {                               // the weights are nobody's output: they are on their way
                pdl_wait();                              // before the kernel that writes the activations has ended
                waited = true;
            }
#pragma unroll
            for (int u = 0; u < DR_U; ++u) {
                const int piece = (s * DR_U + u) * 4 + t;
                av[0][u] = (piece < pieces && lo_ok) ? load_after_wait(a_lo + piece) : zero;
                if (WIDE) av[1][u] = (piece < pieces && hi_ok) ? load_after_wait(a_hi + piece) : zero;
            }
#pragma unroll
            for (int u = 0; u < DR_U; ++u) {
                const uint4 lo = av[0][u], hi = WIDE ? av[1][u] : zero;
#pragma unroll
                for (int i = 0; i < DR_TILES; ++i) {
                    mma_bf16(c[i], lo.x, hi.x, lo.y, hi.y, wv[i][u].x, wv[i][u].y);
                    mma_bf16(c[i], lo.z, hi.z, lo.w, hi.w, wv[i][u].z, wv[i][u].w);
                }
            }
        }
        // c[i][0..1]: activation row g, weight rows 2t, 2t + 1 of tile i; c[i][2..3]: activation row g + 8
#pragma unroll
        for (int i = 0; i < DR_TILES; ++i) {
            part[warp][i][g][2 * t] = c[i][0];
            part[warp][i][g][2 * t + 1] = c[i][1];
            if (WIDE) {
                part[warp][i][g + 8][2 * t] = c[i][2];
                part[warp][i][g + 8][2 * t + 1] = c[i][3];
            }
        }
        __syncthreads();
        constexpr int OUT_TILES = MODE == DR_SWIGLU ? DR_TILES / 2 : DR_TILES;
        for (int o = threadIdx.x; o < OUT_TILES * ROWS * DR_TILE; o += DR_THREADS) {
            const int i = o / (ROWS * DR_TILE), m = (o / DR_TILE) % ROWS, jn = o % DR_TILE;
            const int n = r0 + i * DR_TILE + jn;
            if (m < p.M && n < r_end) {
                float v = 0.0f, v_up = 0.0f;
#pragma unroll
                for (int w = 0; w < DR_WARPS; ++w) {
                    v += part[w][i][m][jn];
                    if (MODE == DR_SWIGLU) v_up += part[w][i + DR_TILES / 2][m][jn];
                }
                if (MODE == DR_SWIGLU) {
                    reinterpret_cast<bf16*>(p.out)[(size_t)m * n_out + n] =
                        __float2bfloat16_rn(v / (1.0f + expf(-v)) * v_up);
                } else {
                    float* dst = reinterpret_cast<float*>(p.out) + (size_t)m * p.N + n;
                    if (MODE == DR_ADD) atomicAdd(dst, v);
                    else *dst = p.bias ? v + p.bias[n] : v;
                }
            }
        }
        __syncthreads();
    }
    if (!waited) pdl_wait();
}

template <int MODE, bool WIDE, int TILES, int U>
int launch_variant(const DenseRowsParams& p, int sms, cudaStream_t stream) {
    // CTAs that are resident at once: the rows are dealt over exactly that many, so there is one wave
    static int resident = 0;
    if (resident == 0) {
        int per_sm = 0;
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, dense_rows_kernel<MODE, WIDE, TILES, U>, DR_THREADS,
                                                          0) != cudaSuccess || per_sm <= 0)
            return SHARPI_LAUNCH_FAILED;
        resident = sms * (per_sm < DR_CTAS_PER_SM ? per_sm : DR_CTAS_PER_SM);
    }
    const int n_out = MODE == DR_SWIGLU ? p.N / 2 : p.N;
    const int grid = resident < n_out ? resident : n_out;
    // Launched the plain way: started early (programmatic dependent launch), its CTAs sit on every SM with all
    // the registers while the kernel before it is still at work, and a decode step came out slower (Scout sizes,
    // 8 layers, batch 1, qkv and o on this kernel: 568 against 617 tok/s), although between two small kernels
    // the early start saves 1.5 us.  The kernel after this one may still start early (pdl_wait signals it).
    dense_rows_kernel<MODE, WIDE, TILES, U><<<grid, DR_THREADS, 0, stream>>>(p);
    SHARPI_CHECK_LAUNCH();
    return SHARPI_OK;
}

// Which shape of the kernel: a CTA should take its rows in one pass (a second, nearly empty group costs a whole
// walk over K), with runs of 256 bytes per row where three tiles are enough for that and 192 bytes with four
// (measured on B200 at 5120 x 5120, 5120 x 8192 and 7168 x 5120: 9.9 / 14.8 / 15.6 us with three tiles of
// four pieces, 10.7 / 16.5 / 12.8 us with four tiles of three; the last has 25 rows per CTA).
template <int MODE, bool WIDE>
int launch_dense_rows(const DenseRowsParams& p, cudaStream_t stream) {
    static int sms = 0;
    if (sms == 0) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess ||
            cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
            return SHARPI_LAUNCH_FAILED;
    }
    if (MODE != DR_SWIGLU) {
        const int slots = sms * DR_CTAS_PER_SM;
        if ((p.N + slots - 1) / slots <= 3 * DR_TILE) return launch_variant<MODE == DR_SWIGLU ? DR_STORE : MODE, WIDE, 3, 4>(p, sms, stream);
    }
    return launch_variant<MODE, WIDE, 4, 3>(p, sms, stream);
}

}  // namespace

// A [M, K] bf16 (1 <= M <= 16), W [N, K] bf16, K a multiple of 8, both 16-byte aligned.
// mode 0: out fp32 [M, N] = A W^T (+ bias); 1: out += A W^T with reductions; 2: N = 2 I, out bf16 [M, I] =
// silu(A Wg^T) * (A Wu^T) with Wg the first I rows of W and Wu the rest.
SHARPI_API int sharpi_dense_rows(const void* A, const void* W, const float* bias, void* out, int M, int N, int K,
                                 int mode, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return SHARPI_OK;
    if (M > 16 || K <= 0 || K % 8 != 0) return SHARPI_BAD_ARGUMENT;
    if (mode == DR_SWIGLU && N % 2 != 0) return SHARPI_BAD_ARGUMENT;
    if (mode != DR_STORE && bias) return SHARPI_BAD_ARGUMENT;
    if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(W)) & 15) return SHARPI_UNALIGNED;
    DenseRowsParams p;
    p.A = reinterpret_cast<const bf16*>(A); p.W = reinterpret_cast<const bf16*>(W); p.bias = bias; p.out = out;
    p.M = M; p.N = N; p.K = K;
    const bool wide = M > 8;
    switch (mode) {
        case DR_STORE: return wide ? launch_dense_rows<DR_STORE, true>(p, stream) : launch_dense_rows<DR_STORE, false>(p, stream);
        case DR_ADD: return wide ? launch_dense_rows<DR_ADD, true>(p, stream) : launch_dense_rows<DR_ADD, false>(p, stream);
        case DR_SWIGLU: return wide ? launch_dense_rows<DR_SWIGLU, true>(p, stream) : launch_dense_rows<DR_SWIGLU, false>(p, stream);
        default: return SHARPI_BAD_ARGUMENT;
    }
}
