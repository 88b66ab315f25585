// Paged attention for portions of prompts (many query rows per request), bf16 cache.
//
// One CTA takes one query head and one tile of up to 64 consecutive rows of one request; its four
// warps own 16 rows each.  It walks the keys the tile may see in blocks of 64, at absolute
// multiples of 64 positions, through the request's block table: keys and values go to shared
// memory with cp.async (two stages), QK^T and PV run on the tensor cores (m16n8k16) with an online
// softmax in fp32 registers.  Masks: causal, plus "same chunk" or "within the window" per element,
// as defined by visible_lo in common.cuh.  A row's result depends on its own position and keys
// only (the key blocks are anchored at absolute positions), not on how the prompt was cut.
//
// Reference counterparts: llm_flash_attn_prefill_tc / _tc2 (16-query tiles per warp, 16-key tiles,
// f16 mma.sync, contiguous per-sequence cache, causal + optional window;
// src/SharpInference.Cuda/CudaTextKernels.cs:7657, :8086-8110).  Differences: the cache is paged,
// the chunk mask exists, keys are bf16, and tiles come from a list so that portions of several
// requests share one launch.
#include "common.cuh"
#include "mma_sync.cuh"

using namespace mma16;

constexpr int PF_BQ = 64;        // query rows per CTA
constexpr int PF_BK = 64;        // keys per block
constexpr int PF_THREADS = 128;

struct PrefillArgs {
    const bf16* q;            // [T, nq, D]
    const bf16* kv;           // [pages, 2, nkv, page_size, D]
    const int* block_table;   // [B, max_blocks]
    const int* tiles;         // [n_tiles, 4]: first row, rows, first position, request index
    bf16* out;                // [T, nq * D]
    int nq, nkv, max_blocks, page_size, mask_kind, mask_span;
    float scale_log2;
};

template <int D>
__device__ __forceinline__ void load_kv_block(const PrefillArgs& a, const int* table, int kvh, int key0, int key_lo,
                                              int key_hi, bf16* k_s, bf16* v_s) {
    constexpr int LD = D + 8, VEC = D / 8;
    const size_t plane = (size_t)a.nkv * a.page_size * D;
    for (int idx = threadIdx.x; idx < PF_BK * VEC; idx += PF_THREADS) {
        const int row = idx / VEC, col = idx % VEC;
        const int key = key0 + row;
        bool valid = key >= key_lo && key <= key_hi;
        const int page = valid ? table[key / a.page_size] : -1;
        valid = valid && page >= 0;
        const bf16* src = a.kv;
        if (valid) src = a.kv + (size_t)page * 2 * plane + ((size_t)kvh * a.page_size + key % a.page_size) * D + col * 8;
        cp_async_16(k_s + row * LD + col * 8, src, valid ? 16 : 0);
        cp_async_16(v_s + row * LD + col * 8, valid ? src + plane : src, valid ? 16 : 0);
    }
}

template <int D>
__global__ void __launch_bounds__(PF_THREADS, 2) attn_prefill_kernel(PrefillArgs a) {
    constexpr int LD = D + 8, VEC = D / 8;
    extern __shared__ __align__(16) uint8_t smem_bytes[];
    bf16* q_s = reinterpret_cast<bf16*>(smem_bytes);     // [64][LD]
    bf16* kv_s = q_s + PF_BQ * LD;                         // [2 stages][K|V][64][LD]

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // the head is the grid's fast index and the last tiles (the ones with the most keys) come first, so that
    // every head's longest tiles start first and the short ones fill the tail
    const int* tile = a.tiles + (size_t)(gridDim.y - 1 - blockIdx.y) * 4;
    const int row0 = tile[0], n_rows = tile[1], p0 = tile[2];
    const int* table = a.block_table + (size_t)tile[3] * a.max_blocks;
    const int head = blockIdx.x;
    const int kvh = head / (a.nq / a.nkv);

    const int p_last = p0 + n_rows - 1;
    const int key_lo = visible_lo(p0, a.mask_kind, a.mask_span);   // lowest key any row of the tile sees
    const int kb_first = key_lo / PF_BK, kb_last = p_last / PF_BK;

    // queries (rows beyond the tile are zero) and the first key block
    for (int idx = threadIdx.x; idx < PF_BQ * VEC; idx += PF_THREADS) {
        const int r = idx / VEC, c = idx % VEC;
        const bool valid = r < n_rows;
        const bf16* src = valid ? a.q + ((size_t)(row0 + r) * a.nq + head) * D + c * 8 : a.q;
        cp_async_16(q_s + r * LD + c * 8, src, valid ? 16 : 0);
    }
    load_kv_block<D>(a, table, kvh, kb_first * PF_BK, key_lo, p_last, kv_s, kv_s + PF_BK * LD);
    cp_async_commit();

    uint32_t qa[D / 16][4];
    float o[D / 8][4];
#pragma unroll
    for (int i = 0; i < D / 8; ++i)
#pragma unroll
        for (int e = 0; e < 4; ++e) o[i][e] = 0.0f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.0f, 0.0f};

    // positions and lowest visible keys of this thread's two rows
    int pos_r[2], lo_r[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        pos_r[h] = p0 + warp * 16 + lane / 4 + 8 * h;
        lo_r[h] = visible_lo(pos_r[h], a.mask_kind, a.mask_span);
    }
    const int warp_pos_hi = p0 + warp * 16 + 15;          // highest position among this warp's rows

    for (int kb = kb_first; kb <= kb_last; ++kb) {
        const int stage = (kb - kb_first) & 1;
        bf16* k_s = kv_s + (size_t)stage * 2 * PF_BK * LD;
        bf16* v_s = k_s + PF_BK * LD;
        if (kb < kb_last) {
            bf16* nk = kv_s + (size_t)(stage ^ 1) * 2 * PF_BK * LD;
            load_kv_block<D>(a, table, kvh, (kb + 1) * PF_BK, key_lo, p_last, nk, nk + PF_BK * LD);
            cp_async_commit();
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        if (kb == kb_first) {
#pragma unroll
            for (int ks = 0; ks < D / 16; ++ks)
                ldmatrix_x4(qa[ks], q_s + (warp * 16 + lane % 16) * LD + ks * 16 + (lane / 16) * 8);
        }
        const int key0 = kb * PF_BK;
        // a warp whose rows all lie below this block (causal) or beyond their window has nothing to do here
        const bool warp_active = key0 <= warp_pos_hi && warp * 16 < n_rows;
        if (warp_active) {
            float s[PF_BK / 8][4];
#pragma unroll
            for (int nt = 0; nt < PF_BK / 8; ++nt) {
#pragma unroll
                for (int e = 0; e < 4; ++e) s[nt][e] = 0.0f;
#pragma unroll
                for (int k2 = 0; k2 < D / 32; ++k2) {
                    uint32_t b[4];
                    ldmatrix_x4(b, k_s + (nt * 8 + (lane % 8)) * LD + k2 * 32 + (lane / 8) * 8);
                    mma_bf16(s[nt], qa[2 * k2], b[0], b[1]);
                    mma_bf16(s[nt], qa[2 * k2 + 1], b[2], b[3]);
                }
                if (D % 32 != 0) {
                    uint32_t b[2];
                    ldmatrix_x2(b, k_s + (nt * 8 + (lane % 8)) * LD + (D - 16) + ((lane / 8) % 2) * 8);
                    mma_bf16(s[nt], qa[D / 16 - 1], b[0], b[1]);
                }
            }
            float m_c[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int nt = 0; nt < PF_BK / 8; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int key = key0 + nt * 8 + (lane % 4) * 2 + (e & 1);
                    const int h = e >> 1;
                    const bool valid = key <= pos_r[h] && key >= lo_r[h];
                    s[nt][e] = valid ? s[nt][e] * a.scale_log2 : -INFINITY;
                    m_c[h] = fmaxf(m_c[h], s[nt][e]);
                }
            float corr[2], l_c[2] = {0.0f, 0.0f};
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                m_c[h] = fmaxf(m_c[h], __shfl_xor_sync(0xffffffffu, m_c[h], 1));
                m_c[h] = fmaxf(m_c[h], __shfl_xor_sync(0xffffffffu, m_c[h], 2));
                const float m_new = fmaxf(m_run[h], m_c[h]);
                corr[h] = (m_run[h] == -INFINITY) ? 0.0f : exp2f(m_run[h] - m_new);
                m_run[h] = m_new;
            }
#pragma unroll
            for (int nt = 0; nt < PF_BK / 8; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float p = (s[nt][e] == -INFINITY) ? 0.0f : exp2f(s[nt][e] - m_run[e >> 1]);
                    s[nt][e] = p;
                    l_c[e >> 1] += p;
                }
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                l_c[h] += __shfl_xor_sync(0xffffffffu, l_c[h], 1);
                l_c[h] += __shfl_xor_sync(0xffffffffu, l_c[h], 2);
                l_run[h] = l_run[h] * corr[h] + l_c[h];
            }
#pragma unroll
            for (int i = 0; i < D / 8; ++i) {
                o[i][0] *= corr[0]; o[i][1] *= corr[0];
                o[i][2] *= corr[1]; o[i][3] *= corr[1];
            }
#pragma unroll
            for (int j = 0; j < PF_BK / 16; ++j) {
                uint32_t pa[4];
                pa[0] = pack_bf16(s[2 * j][0], s[2 * j][1]);
                pa[1] = pack_bf16(s[2 * j][2], s[2 * j][3]);
                pa[2] = pack_bf16(s[2 * j + 1][0], s[2 * j + 1][1]);
                pa[3] = pack_bf16(s[2 * j + 1][2], s[2 * j + 1][3]);
#pragma unroll
                for (int d2 = 0; d2 < D / 16; ++d2) {
                    uint32_t b[4];
                    ldmatrix_x4_trans(b, v_s + (j * 16 + (lane % 8) + ((lane / 8) % 2) * 8) * LD + d2 * 16 + (lane / 16) * 8);
                    mma_bf16(o[2 * d2], pa, b[0], b[1]);
                    mma_bf16(o[2 * d2 + 1], pa, b[2], b[3]);
                }
            }
        }
        __syncthreads();   // the other stage is overwritten by the next iteration's loads
    }

#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int r = warp * 16 + lane / 4 + 8 * h;
        if (r < n_rows) {
            const float inv = 1.0f / l_run[h];
            bf16* dst = a.out + ((size_t)(row0 + r) * a.nq + head) * D + (lane % 4) * 2;
#pragma unroll
            for (int i = 0; i < D / 8; ++i) {
                *reinterpret_cast<__nv_bfloat162*>(dst + i * 8) =
                    __floats2bfloat162_rn(o[i][2 * h] * inv, o[i][2 * h + 1] * inv);
            }
        }
    }
}

template <int D>
static int launch_prefill(const PrefillArgs& a, int n_tiles, cudaStream_t stream) {
    constexpr int LD = D + 8;
    constexpr int SMEM = (PF_BQ * LD + 2 * 2 * PF_BK * LD) * 2;
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(attn_prefill_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM) != cudaSuccess)
            return SHARPI_LAUNCH_FAILED;
        configured = true;
    }
    attn_prefill_kernel<D><<<dim3(a.nq, n_tiles), PF_THREADS, SMEM, stream>>>(a);
    SHARPI_CHECK_LAUNCH();
    return SHARPI_OK;
}

SHARPI_API int sharpi_attention_prefill(const void* q, const void* kv, const int* block_table, const int* tiles,
                                        void* out, int n_tiles, int nq, int nkv, int d, int max_blocks, int page_size,
                                        int mask_kind, int mask_span, float scale, cudaStream_t stream) {
    if (n_tiles <= 0) return SHARPI_OK;
    if (n_tiles > 65535) return SHARPI_BAD_ARGUMENT;        // tiles are the grid's second extent
    if (nq <= 0 || nkv <= 0 || nq % nkv != 0 || page_size <= 0 || max_blocks <= 0 || nq > 65535)
        return SHARPI_BAD_ARGUMENT;
    if (mask_kind != SHARPI_MASK_FULL && mask_span <= 0) return SHARPI_BAD_ARGUMENT;
    if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(kv) | reinterpret_cast<uintptr_t>(out)) & 15)
        return SHARPI_UNALIGNED;
    PrefillArgs a;
    a.q = (const bf16*)q; a.kv = (const bf16*)kv; a.block_table = block_table; a.tiles = tiles; a.out = (bf16*)out;
    a.nq = nq; a.nkv = nkv; a.max_blocks = max_blocks; a.page_size = page_size; a.mask_kind = mask_kind;
    a.mask_span = mask_span; a.scale_log2 = scale * 1.4426950408889634f;
    switch (d) {
        case 16: return launch_prefill<16>(a, n_tiles, stream);
        case 32: return launch_prefill<32>(a, n_tiles, stream);
        case 48: return launch_prefill<48>(a, n_tiles, stream);
        case 64: return launch_prefill<64>(a, n_tiles, stream);
        case 80: return launch_prefill<80>(a, n_tiles, stream);
        case 96: return launch_prefill<96>(a, n_tiles, stream);
        case 112: return launch_prefill<112>(a, n_tiles, stream);
        case 128: return launch_prefill<128>(a, n_tiles, stream);
        default: return SHARPI_BAD_ARGUMENT;   // other head sizes use the generic kernel
    }
}
