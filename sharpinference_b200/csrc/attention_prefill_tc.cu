// Paged attention for portions of prompts on the 5th-generation tensor cores: QK^T and PV are
// tcgen05.mma with the scores S and the per-block outputs O in tensor memory, the query tile, the
// key and value blocks and the probabilities P in shared memory, keys and values fetched page by
// page with TMA.  One CTA serves one query head and a tile of up to 128 consecutive rows of one
// request; a softmax thread owns one row, so row maxima and sums need no shuffles.
//
//   warps 0-3  softmax: read S (tcgen05.ld), mask, exp2, running max / sum, write P (bf16, swizzled)
//              to shared memory, then fold the previous block's O into the row's fp32 accumulator
//   warp 4     TMA producer: Q once, then K and V blocks of 64 keys through the block table
//   warp 5     allocates tensor memory, issues the MMAs: S[j] = Q K_j^T, then O[j-1] = P[j-1] V[j-1]
//
// S, P and O are double-buffered, so QK^T of block j+1 runs while block j is in softmax.  Key blocks
// sit at absolute multiples of 64 positions: a row's result depends on its own position and keys only.
// Every wait is bounded; a wait that gives up records a code in *status and the kernel winds down.
//
// Sizes: head size 64 or 128, pages of a multiple of 64 positions, bf16.  Everything else takes the
// warp-level kernel (attention_prefill.cu) or the generic one.  The reference's counterparts are the
// f16 mma.sync prefill kernels (src/SharpInference.Cuda/CudaTextKernels.cs:7657, :8086-8110).
#include "common.cuh"
#include "sm100.cuh"
#include "tensor_map.cuh"

#include <string.h>

using namespace sm100;

constexpr int TQ = 128;        // query rows per CTA (MMA M)
constexpr int TK = 64;         // keys per block
constexpr int TC_ATT_THREADS = 192;
constexpr int KV_STAGES = 3;

struct PrefillTcArgs {
    const int* block_table;   // [B, max_blocks]
    const int* tiles;         // [n_tiles, 4]: first row, rows, first position, request index
    bf16* out;                // [T, nq * D]
    int* status;
    int nq, nkv, max_blocks, page_size, page_shift, mask_kind, mask_span;
    float scale_log2;
};

enum { ERR_Q = 11, ERR_K = 12, ERR_V = 13, ERR_S = 14, ERR_P = 15, ERR_O = 16, ERR_EMPTY = 17, ERR_ALIGN = 18 };

template <int D>
struct AttCfg {
    static constexpr int HALVES = D / 64;
    static constexpr int Q_BYTES = TQ * D * 2;
    static constexpr int KV_BYTES = TK * D * 2;           // one K or V block
    static constexpr int P_BYTES = TQ * TK * 2;
    static constexpr int SMEM = Q_BYTES + 2 * KV_STAGES * KV_BYTES + 2 * P_BYTES + 1024 + 512;
    static constexpr int S_COL = 0;                        // S[2]: 64 columns each
    static constexpr int O_COL = 2 * TK;                   // O[2]: D columns each
    static constexpr int TMEM_COLS = (2 * TK + 2 * D) <= 256 ? 256 : 512;
};

template <int D>
__global__ void __launch_bounds__(TC_ATT_THREADS, 1)
attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap q_map, const __grid_constant__ CUtensorMap kv_map,
                       const PrefillTcArgs a) {
    using Cfg = AttCfg<D>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* q_s = smem;
    uint8_t* k_s = q_s + Cfg::Q_BYTES;                          // [stages][halves][64 keys][64]
    uint8_t* v_s = k_s + KV_STAGES * Cfg::KV_BYTES;
    uint8_t* p_s = v_s + KV_STAGES * Cfg::KV_BYTES;             // [2][128 rows][64 keys]
    uint64_t* bars = reinterpret_cast<uint64_t*>(p_s + 2 * Cfg::P_BYTES);
    uint64_t* q_full = bars;
    uint64_t* k_full = bars + 1;
    uint64_t* k_empty = k_full + KV_STAGES;
    uint64_t* v_full = k_empty + KV_STAGES;
    uint64_t* v_empty = v_full + KV_STAGES;
    uint64_t* s_full = v_empty + KV_STAGES;       // [2]
    uint64_t* p_full = s_full + 2;                // [2] 128 arrivals
    uint64_t* p_empty = p_full + 2;               // [2]
    uint64_t* o_full = p_empty + 2;               // [2]
    uint64_t* o_empty = o_full + 2;               // [2] 128 arrivals
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(o_empty + 2);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int* tile = a.tiles + (size_t)blockIdx.x * 4;
    const int row0 = tile[0], n_rows = tile[1], p0 = tile[2];
    const int* table = a.block_table + (size_t)tile[3] * a.max_blocks;
    const int head = blockIdx.y;
    const int kvh = head / (a.nq / a.nkv);
    const int p_last = p0 + n_rows - 1;
    const int key_lo = visible_lo(p0, a.mask_kind, a.mask_span);
    const int kb_first = key_lo / TK, n_blocks = p_last / TK - kb_first + 1;

    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        for (int s = 0; s < KV_STAGES; ++s) {
            mbar_init(&k_full[s], 1); mbar_init(&k_empty[s], 1);
            mbar_init(&v_full[s], 1); mbar_init(&v_empty[s], 1);
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(&s_full[s], 1); mbar_init(&p_full[s], 128); mbar_init(&p_empty[s], 1);
            mbar_init(&o_full[s], 1); mbar_init(&o_empty[s], 128);
        }
        fence_barrier_init();
    }
    if (warp == 5) {
        tmem_alloc(tmem_slot, Cfg::TMEM_COLS);
        tmem_relinquish();
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 4) {
        // ---- TMA producer ----------------------------------------------------------------------
        if (lane == 0) {
            prefetch_tensormap(&q_map);
            prefetch_tensormap(&kv_map);
            mbar_arrive_expect_tx(q_full, Cfg::Q_BYTES);
#pragma unroll
            for (int hf = 0; hf < Cfg::HALVES; ++hf)
                tma_load_2d(q_s + hf * TQ * 128, &q_map, q_full, head * D + hf * 64, row0);
            bool ok = true;
            for (int j = 0; j < n_blocks && ok; ++j) {
                const int st = j % KV_STAGES, use = j / KV_STAGES;
                const int key0 = (kb_first + j) * TK;
                const int blk = key0 >> a.page_shift;
                const int page = table[blk];
                const int off = key0 - (blk << a.page_shift);
                const int row_k = ((page * 2 + 0) * a.nkv + kvh) * a.page_size + off;
                const int row_v = ((page * 2 + 1) * a.nkv + kvh) * a.page_size + off;
                if (use > 0) ok = mbar_wait(&k_empty[st], (use - 1) & 1);
                if (!ok) { atomicExch(a.status, ERR_EMPTY); break; }
                mbar_arrive_expect_tx(&k_full[st], Cfg::KV_BYTES);
#pragma unroll
                for (int hf = 0; hf < Cfg::HALVES; ++hf)
                    tma_load_2d(k_s + st * Cfg::KV_BYTES + hf * TK * 128, &kv_map, &k_full[st], hf * 64, row_k);
                if (use > 0) ok = mbar_wait(&v_empty[st], (use - 1) & 1);
                if (!ok) { atomicExch(a.status, ERR_EMPTY); break; }
                mbar_arrive_expect_tx(&v_full[st], Cfg::KV_BYTES);
#pragma unroll
                for (int hf = 0; hf < Cfg::HALVES; ++hf)
                    tma_load_2d(v_s + st * Cfg::KV_BYTES + hf * TK * 128, &kv_map, &v_full[st], hf * 64, row_v);
            }
        }
    } else if (warp == 5) {
        // ---- MMA issuer ------------------------------------------------------------------------
        if (lane == 0) {
            const uint32_t idesc_qk = instr_desc_bf16(TQ, TK);
            const uint32_t idesc_pv = instr_desc_bf16(TQ, D, true);
            bool ok = mbar_wait(q_full, 0);
            if (!ok) atomicExch(a.status, ERR_Q);
            auto pv = [&](int i) -> bool {
                const int st = i % KV_STAGES, b = i & 1;
                if (!mbar_wait(&p_full[b], (i >> 1) & 1)) { atomicExch(a.status, ERR_P); return false; }
                if (!mbar_wait(&v_full[st], (i / KV_STAGES) & 1)) { atomicExch(a.status, ERR_V); return false; }
                if (i >= 2 && !mbar_wait(&o_empty[b], ((i >> 1) - 1) & 1)) { atomicExch(a.status, ERR_O); return false; }
                tcgen05_fence_after();
                const uint8_t* pt = p_s + b * Cfg::P_BYTES;
                const uint8_t* vt = v_s + st * Cfg::KV_BYTES;
#pragma unroll
                for (int ks = 0; ks < TK / 16; ++ks)
                    mma_bf16_ss(tmem_base + Cfg::O_COL + b * D, smem_desc_k_sw128(pt, ks * 32),
                                smem_desc_mn_sw128(vt, TK * 128, ks * 2048), idesc_pv, ks != 0);
                mma_commit(&v_empty[st]);
                mma_commit(&p_empty[b]);
                mma_commit(&o_full[b]);
                return true;
            };
            for (int j = 0; j < n_blocks && ok; ++j) {
                const int st = j % KV_STAGES;
                ok = mbar_wait(&k_full[st], (j / KV_STAGES) & 1);
                if (!ok) { atomicExch(a.status, ERR_K); break; }
                tcgen05_fence_after();
                const uint8_t* kt = k_s + st * Cfg::KV_BYTES;
#pragma unroll
                for (int ks = 0; ks < D / 16; ++ks)
                    mma_bf16_ss(tmem_base + Cfg::S_COL + (j & 1) * TK,
                                smem_desc_k_sw128(q_s + (ks / 4) * TQ * 128, (ks % 4) * 32),
                                smem_desc_k_sw128(kt + (ks / 4) * TK * 128, (ks % 4) * 32), idesc_qk, ks != 0);
                mma_commit(&k_empty[st]);
                mma_commit(&s_full[j & 1]);
                if (j >= 1) ok = pv(j - 1);
            }
            if (ok) pv(n_blocks - 1);
        }
    } else {
        // ---- softmax: thread = query row ---------------------------------------------------------
        const int r = warp * 32 + lane;
        const int pos_r = p0 + r;
        const int lo_r = visible_lo(pos_r, a.mask_kind, a.mask_span);
        const uint32_t lane_addr = tmem_base + ((uint32_t)(warp * 32) << 16);
        float o[D];
#pragma unroll
        for (int i = 0; i < D; ++i) o[i] = 0.0f;
        float m_run = -INFINITY, l_run = 0.0f, corr_prev = 1.0f;
        bool ok = true;

        auto fold = [&](int i, float corr) -> bool {       // o = o * corr + O_i
            const int b = i & 1;
            if (!mbar_wait(&o_full[b], (i >> 1) & 1)) { atomicExch(a.status, ERR_O); return false; }
            tcgen05_fence_after();
#pragma unroll
            for (int c0 = 0; c0 < D; c0 += 32) {
                uint32_t v[32];
                tmem_ld_32_nowait(lane_addr + Cfg::O_COL + b * D + c0, v);
                tmem_ld_wait();
#pragma unroll
                for (int i2 = 0; i2 < 32; ++i2) o[c0 + i2] = fmaf(o[c0 + i2], corr, __uint_as_float(v[i2]));
            }
            tcgen05_fence_before();
            mbar_arrive(&o_empty[b]);
            return true;
        };

        for (int j = 0; j < n_blocks; ++j) {
            const int b = j & 1;
            if (!mbar_wait(&s_full[b], (j >> 1) & 1)) { atomicExch(a.status, ERR_S); ok = false; break; }
            tcgen05_fence_after();
            uint32_t sv[TK];
            tmem_ld_32_nowait(lane_addr + Cfg::S_COL + b * TK, sv);
            tmem_ld_32_nowait(lane_addr + Cfg::S_COL + b * TK + 32, sv + 32);
            tmem_ld_wait();
            const int key0 = (kb_first + j) * TK;
            float m_blk = -INFINITY;
#pragma unroll
            for (int c = 0; c < TK; ++c) {
                const int key = key0 + c;
                const float s = (key <= pos_r && key >= lo_r) ? __uint_as_float(sv[c]) * a.scale_log2 : -INFINITY;
                sv[c] = __float_as_uint(s);
                m_blk = fmaxf(m_blk, s);
            }
            const float m_new = fmaxf(m_run, m_blk);
            const float corr = (m_run == -INFINITY) ? 1.0f : exp2f(m_run - m_new);   // nothing accumulated yet: any factor
            float l_blk = 0.0f;
            uint32_t packed[TK / 2];
#pragma unroll
            for (int c = 0; c < TK; c += 2) {
                const float s0 = __uint_as_float(sv[c]), s1 = __uint_as_float(sv[c + 1]);
                const float e0 = (s0 == -INFINITY) ? 0.0f : exp2f(s0 - m_new);
                const float e1 = (s1 == -INFINITY) ? 0.0f : exp2f(s1 - m_new);
                l_blk += e0 + e1;
                __nv_bfloat162 pr = __floats2bfloat162_rn(e0, e1);
                packed[c / 2] = *reinterpret_cast<uint32_t*>(&pr);
            }
            l_run = l_run * corr + l_blk;
            m_run = m_new;
            // P[b] may be overwritten once the MMAs that read it two blocks ago are done
            if (j >= 2 && !mbar_wait(&p_empty[b], ((j >> 1) - 1) & 1)) { atomicExch(a.status, ERR_P); ok = false; break; }
            uint8_t* prow = p_s + b * Cfg::P_BYTES + r * 128;
#pragma unroll
            for (int ch = 0; ch < 8; ++ch)
                *reinterpret_cast<uint4*>(prow + ((ch ^ (r & 7)) << 4)) =
                    make_uint4(packed[ch * 4], packed[ch * 4 + 1], packed[ch * 4 + 2], packed[ch * 4 + 3]);
            fence_proxy_async();
            tcgen05_fence_before();
            mbar_arrive(&p_full[b]);
            if (j >= 1 && !fold(j - 1, corr_prev)) { ok = false; break; }
            corr_prev = corr;
        }
        if (ok) ok = fold(n_blocks - 1, corr_prev);
        if (ok && r < n_rows) {
            const float inv = 1.0f / l_run;
            bf16* dst = a.out + ((size_t)(row0 + r) * a.nq + head) * D;
#pragma unroll
            for (int c = 0; c < D; c += 8) {
                uint4 w;
                __nv_bfloat162 h0 = __floats2bfloat162_rn(o[c] * inv, o[c + 1] * inv);
                __nv_bfloat162 h1 = __floats2bfloat162_rn(o[c + 2] * inv, o[c + 3] * inv);
                __nv_bfloat162 h2 = __floats2bfloat162_rn(o[c + 4] * inv, o[c + 5] * inv);
                __nv_bfloat162 h3 = __floats2bfloat162_rn(o[c + 6] * inv, o[c + 7] * inv);
                w.x = *reinterpret_cast<uint32_t*>(&h0); w.y = *reinterpret_cast<uint32_t*>(&h1);
                w.z = *reinterpret_cast<uint32_t*>(&h2); w.w = *reinterpret_cast<uint32_t*>(&h3);
                *reinterpret_cast<uint4*>(dst + c) = w;
            }
        }
    }
    tcgen05_fence_before();
    __syncthreads();
    if (warp == 5) {
        tcgen05_fence_after();
        tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
    }
}

template <int D>
static int launch_tc(const CUtensorMap& qm, const CUtensorMap& kvm, const PrefillTcArgs& a, int n_tiles, cudaStream_t stream) {
    using Cfg = AttCfg<D>;
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(attn_prefill_tc_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM) !=
            cudaSuccess)
            return SHARPI_LAUNCH_FAILED;
        configured = true;
    }
    attn_prefill_tc_kernel<D><<<dim3(n_tiles, a.nq), TC_ATT_THREADS, Cfg::SMEM, stream>>>(qm, kvm, a);
    SHARPI_CHECK_LAUNCH();
    return SHARPI_OK;
}

// q [T, nq, d] bf16; kv [num_pages, 2, nkv, page_size, d] bf16; tiles of up to 128 rows.
SHARPI_API int sharpi_attention_prefill_tc(const void* q, const void* kv, const int* block_table, const int* tiles,
                                           void* out, int* status, int T, int num_pages, int n_tiles, int nq, int nkv,
                                           int d, int max_blocks, int page_size, int mask_kind, int mask_span,
                                           float scale, cudaStream_t stream) {
    if (n_tiles <= 0) return SHARPI_OK;
    if (nq <= 0 || nkv <= 0 || nq % nkv != 0 || max_blocks <= 0 || nq > 65535 || !status) return SHARPI_BAD_ARGUMENT;
    if (d != 64 && d != 128) return SHARPI_BAD_ARGUMENT;
    if (page_size < 64 || (page_size & (page_size - 1)) != 0) return SHARPI_BAD_ARGUMENT;
    if (mask_kind != SHARPI_MASK_FULL && mask_span <= 0) return SHARPI_BAD_ARGUMENT;
    if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(kv) | reinterpret_cast<uintptr_t>(out)) & 15)
        return SHARPI_UNALIGNED;
    CUtensorMap qm, kvm;
    if (!tmap::make_bf16_map(&qm, q, (uint64_t)nq * d, (uint64_t)T, 0, 64, TQ)) return SHARPI_LAUNCH_FAILED;
    if (!tmap::make_bf16_map(&kvm, kv, (uint64_t)d, (uint64_t)num_pages * 2 * nkv * page_size, 0, 64, TK))
        return SHARPI_LAUNCH_FAILED;
    PrefillTcArgs a;
    a.block_table = block_table; a.tiles = tiles; a.out = (bf16*)out; a.status = status;
    a.nq = nq; a.nkv = nkv; a.max_blocks = max_blocks; a.page_size = page_size; a.mask_kind = mask_kind;
    a.mask_span = mask_span; a.scale_log2 = scale * 1.4426950408889634f;
    a.page_shift = 0;
    while ((1 << a.page_shift) < page_size) ++a.page_shift;
    if (d == 64) return launch_tc<64>(qm, kvm, a, n_tiles, stream);
    return launch_tc<128>(qm, kvm, a, n_tiles, stream);
}
