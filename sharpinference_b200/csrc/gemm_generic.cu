// C = A . W^T on the CUDA cores with fp32 accumulation, for any M, N, K: the matrix product
// of the true 32-bit path (no tensor cores, no reduced-precision mode) and the fallback for
// shapes the tensor-core kernels refuse.  Dense and grouped (one weight matrix per expert,
// rows sorted by expert) share the kernel.
//
// Each output element is one chain of fused multiply-adds over k = 0 .. K-1 in order, so its
// value depends on its own row and column only: never on M, on the other rows of the step or
// on the tile it fell into.  The reference's counterparts are llm_matvec_f32
// (src/SharpInference.Cuda/CudaTextKernels.cs:1325) and its per-expert matvec loop
// (src/SharpInference.Engine/CudaForwardPass.cs:5554-5578).
#include "common.cuh"

constexpr int GB_M = 64, GB_N = 64, GB_K = 16;

struct GemmArgs {
    const void* A;              // [rows, K], row r of the product reads A[a_rows ? a_rows[r] : r]
    const void* W;              // [E, N, K]
    float* C;                   // [rows, N], row r writes C[out_rows ? out_rows[r] : r]
    const int* group_offsets;   // [E + 1] first sorted row of every group; null: one group [0, M)
    const int* a_rows;
    const int* out_rows;
    int M, N, K, E;
    int accumulate;             // C += instead of C =
    const float* bias;          // [N] added to every row (nullable)
    const float* row_scale;     // row r of the product is multiplied by row_scale[scale_rows ? scale_rows[r] : r]
    const int* scale_rows;      //   before the bias and before it is stored or added in (both nullable)
};

template <typename TA, typename TW>
__global__ void __launch_bounds__(256) gemm_nt_kernel(GemmArgs g) {
    __shared__ float As[GB_K][GB_M + 4];
    __shared__ float Ws[GB_K][GB_N + 4];

    int m0, m_end, e = 0;
    if (g.group_offsets) {
        int tile = blockIdx.y;
        int start = 0;
        for (; e < g.E; ++e) {
            start = g.group_offsets[e];
            const int n = g.group_offsets[e + 1] - start;
            const int tiles = (n + GB_M - 1) / GB_M;
            if (tile < tiles) break;
            tile -= tiles;
        }
        if (e >= g.E) return;
        m0 = start + tile * GB_M;
        m_end = g.group_offsets[e + 1];
    } else {
        m0 = blockIdx.y * GB_M;
        m_end = g.M;
        if (m0 >= m_end) return;
    }
    const int n0 = blockIdx.x * GB_N;
    const TA* A = (const TA*)g.A;
    const TW* W = (const TW*)g.W + (size_t)e * g.N * g.K;

    const int tid = threadIdx.x;
    const int lrow = tid >> 2;        // 0..63: tile row loaded by this thread
    const int lk = (tid & 3) * 4;     // 0,4,8,12: first of its 4 k values
    const int am = m0 + lrow;
    const bool a_ok = am < m_end;
    const TA* a_ptr = a_ok ? A + (size_t)(g.a_rows ? g.a_rows[am] : am) * g.K : nullptr;
    const int wn = n0 + lrow;
    const bool w_ok = wn < g.N;
    const TW* w_ptr = w_ok ? W + (size_t)wn * g.K : nullptr;

    const int tx = tid & 15, ty = tid >> 4;  // thread computes rows ty*4.., cols tx*4..
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;

    for (int k0 = 0; k0 < g.K; k0 += GB_K) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int k = k0 + lk + i;
            As[lk + i][lrow] = (a_ok && k < g.K) ? to_float(a_ptr[k]) : 0.0f;
            Ws[lk + i][lrow] = (w_ok && k < g.K) ? to_float(w_ptr[k]) : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < GB_K; ++k) {
            float av[4], wv[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) av[i] = As[k][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) wv[j] = Ws[k][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], wv[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int m = m0 + ty * 4 + i;
        if (m >= m_end) continue;
        float* crow = g.C + (size_t)(g.out_rows ? g.out_rows[m] : m) * g.N;
        const float s = g.row_scale ? g.row_scale[g.scale_rows ? g.scale_rows[m] : m] : 1.0f;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n < g.N) {
                float v = g.row_scale ? acc[i][j] * s : acc[i][j];
                if (g.bias) v += g.bias[n];
                crow[n] = g.accumulate ? crow[n] + v : v;
            }
        }
    }
}

SHARPI_API int sharpi_gemm_nt(const void* A, int a_dtype, const void* W, int w_dtype, float* C,
                              const int* group_offsets, const int* a_rows, const int* out_rows, int M, int N,
                              int K, int E, int accumulate, const float* bias, const float* row_scale,
                              const int* scale_rows, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return SHARPI_OK;
    if (K <= 0 || E <= 0) return SHARPI_BAD_ARGUMENT;
    if (!group_offsets && E != 1) return SHARPI_BAD_ARGUMENT;
    GemmArgs g;
    g.A = A; g.W = W; g.C = C; g.group_offsets = group_offsets; g.a_rows = a_rows; g.out_rows = out_rows;
    g.M = M; g.N = N; g.K = K; g.E = E; g.accumulate = accumulate;
    g.bias = bias; g.row_scale = row_scale; g.scale_rows = scale_rows;
    long long m_tiles = (M + GB_M - 1) / GB_M + (group_offsets ? E : 0);
    long long n_tiles = (N + GB_N - 1) / GB_N;
    if (m_tiles > 65535 || n_tiles > 2147483647LL) return SHARPI_BAD_ARGUMENT;
    dim3 grid((unsigned)n_tiles, (unsigned)m_tiles);
    if (a_dtype == SHARPI_F32 && w_dtype == SHARPI_F32)
        gemm_nt_kernel<float, float><<<grid, 256, 0, stream>>>(g);
    else if (a_dtype == SHARPI_BF16 && w_dtype == SHARPI_BF16)
        gemm_nt_kernel<bf16, bf16><<<grid, 256, 0, stream>>>(g);
    else if (a_dtype == SHARPI_F32 && w_dtype == SHARPI_BF16)
        gemm_nt_kernel<float, bf16><<<grid, 256, 0, stream>>>(g);
    else if (a_dtype == SHARPI_BF16 && w_dtype == SHARPI_F32)
        gemm_nt_kernel<bf16, float><<<grid, 256, 0, stream>>>(g);
    else
        return SHARPI_BAD_ARGUMENT;
    SHARPI_CHECK_LAUNCH();
    return SHARPI_OK;
}
