// Paged attention for any head size, head count and grouping, in fp32 or bf16 storage:
// the kernel of the true 32-bit path, and the one every other attention kernel is checked
// against on the device.  One block serves one (token row, query head): it walks the keys
// the row may see in tiles of 128, through the request's block table, with an online
// softmax; scores, maxima, exponentials, sums and the weighted value sum are fp32.
//
// The reference's counterpart is llm_attention (one block per query head, scores in shared
// memory, three-phase softmax, serial value sum; src/SharpInference.Cuda/CudaTextKernels.cs:7384)
// with the score formula of src/SharpInference.Engine/ForwardPass.cs:1850-1911:
// s_t = (q . k_t) / sqrt(d) over the visible t, p = softmax(s), o = sum_t p_t v_t, query head
// h reading kv head h / (nq / nkv).  Chunked and windowed visibility are not in the
// reference; `visible_lo` in common.cuh defines them.
//
// The tiles start at the row's lowest visible position, which depends on the row's own
// position only, so a row's result does not depend on how the step was cut or batched.
#include "common.cuh"

constexpr int ATT_THREADS = 128;
constexpr int ATT_TILE = 128;
constexpr int ATT_MAX_D = 512;

struct PagedAttnArgs {
    const void* q;           // [T, nq, d]
    const void* kv_base;     // [page][2][nkv][page_size][d]
    const int* block_table;  // [B, max_blocks]
    const int* row_req;      // [T]
    const int* positions;    // [T]
    void* out;               // [T, nq * d]
    int T, nq, nkv, d, max_blocks, page_size;
    int mask_kind, mask_span;
    float scale;
};

template <typename TS>
__global__ void paged_attention_generic_kernel(PagedAttnArgs a) {
    __shared__ float q_s[ATT_MAX_D];
    __shared__ float p_s[ATT_TILE];
    __shared__ long long off_s[ATT_TILE];  // element offset of the key row inside the K plane; V adds `plane`
    __shared__ float scratch[32];

    const int t = blockIdx.x;
    const int h = blockIdx.y;
    const int d = a.d;
    const int kvh = h / (a.nq / a.nkv);
    const int pos = a.positions[t];
    const int lo = visible_lo(pos, a.mask_kind, a.mask_span);
    const int* table = a.block_table + (size_t)a.row_req[t] * a.max_blocks;
    const size_t plane = (size_t)a.nkv * a.page_size * d;
    const TS* kv = (const TS*)a.kv_base;

    const TS* qrow = (const TS*)a.q + ((size_t)t * a.nq + h) * d;
    for (int i = threadIdx.x; i < d; i += ATT_THREADS) q_s[i] = to_float(qrow[i]);
    __syncthreads();

    constexpr int DPT = ATT_MAX_D / ATT_THREADS;  // output dims per thread
    float acc[DPT];
#pragma unroll
    for (int r = 0; r < DPT; ++r) acc[r] = 0.0f;
    float m_run = -INFINITY, l_run = 0.0f;

    for (int tile = lo; tile <= pos; tile += ATT_TILE) {
        const int key = tile + threadIdx.x;
        float s = -INFINITY;
        long long off = -1;
        if (key <= pos) {
            const int page = table[key / a.page_size];
            if (page >= 0) {
                off = (long long)page * 2 * plane + ((long long)kvh * a.page_size + key % a.page_size) * d;
                const TS* krow = kv + off;
                float dot = 0.0f;
                for (int i = 0; i < d; ++i) dot += q_s[i] * to_float(krow[i]);
                s = dot * a.scale;
            }
        }
        const float m_tile = block_max(s, scratch);
        const float m_new = fmaxf(m_run, m_tile);
        // m_new is finite: the row's own key is always visible and present.
        const float p = (off >= 0) ? expf(s - m_new) : 0.0f;
        const float corr = (m_run == -INFINITY) ? 0.0f : expf(m_run - m_new);
        __syncthreads();  // the previous tile's p_s / off_s are no longer read
        p_s[threadIdx.x] = p;
        off_s[threadIdx.x] = off;
        const float l_tile = block_sum(p, scratch);  // has __syncthreads inside: p_s/off_s are visible after it
        l_run = l_run * corr + l_tile;
        m_run = m_new;
        const int n_keys = min(ATT_TILE, pos - tile + 1);
#pragma unroll
        for (int r = 0; r < DPT; ++r) {
            const int i = threadIdx.x + r * ATT_THREADS;
            if (i < d) {
                float sum = 0.0f;
                for (int k = 0; k < n_keys; ++k) {
                    const long long o = off_s[k];
                    if (o >= 0) sum += p_s[k] * to_float(kv[o + plane + i]);
                }
                acc[r] = acc[r] * corr + sum;
            }
        }
    }
    TS* orow = (TS*)a.out + ((size_t)t * a.nq + h) * d;
    const float inv_l = 1.0f / l_run;
#pragma unroll
    for (int r = 0; r < DPT; ++r) {
        const int i = threadIdx.x + r * ATT_THREADS;
        if (i < d) orow[i] = from_float<TS>(acc[r] * inv_l);
    }
}

SHARPI_API int sharpi_paged_attention_generic(const void* q, const void* kv_base, const int* block_table,
                                              const int* row_req, const int* positions, void* out, int dtype,
                                              int T, int nq, int nkv, int d, int max_blocks, int page_size,
                                              int mask_kind, int mask_span, float scale, cudaStream_t stream) {
    if (T <= 0) return SHARPI_OK;
    if (nq <= 0 || nkv <= 0 || nq % nkv != 0 || d <= 0 || d > ATT_MAX_D || nq > 65535 || page_size <= 0 ||
        max_blocks <= 0)
        return SHARPI_BAD_ARGUMENT;
    if (mask_kind != SHARPI_MASK_FULL && mask_span <= 0) return SHARPI_BAD_ARGUMENT;
    PagedAttnArgs a;
    a.q = q; a.kv_base = kv_base; a.block_table = block_table; a.row_req = row_req; a.positions = positions;
    a.out = out; a.T = T; a.nq = nq; a.nkv = nkv; a.d = d; a.max_blocks = max_blocks; a.page_size = page_size;
    a.mask_kind = mask_kind; a.mask_span = mask_span; a.scale = scale;
    dim3 grid(T, nq);
    if (dtype == SHARPI_F32)
        paged_attention_generic_kernel<float><<<grid, ATT_THREADS, 0, stream>>>(a);
    else if (dtype == SHARPI_BF16)
        paged_attention_generic_kernel<bf16><<<grid, ATT_THREADS, 0, stream>>>(a);
    else
        return SHARPI_BAD_ARGUMENT;
    SHARPI_CHECK_LAUNCH();
    return SHARPI_OK;
}
