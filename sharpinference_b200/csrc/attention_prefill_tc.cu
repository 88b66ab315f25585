// Paged attention for portions of prompts on the 5th-generation tensor cores: QK^T and PV are
// tcgen05.mma with the scores S and the per-block outputs O in tensor memory, the query tile, the
// key and value blocks and the probabilities P in shared memory, keys and values fetched page by
// page with TMA.  One CTA serves one query head and a tile of up to 128 consecutive rows of one
// request; a softmax thread owns one row, so row maxima and sums need no shuffles.
//
//   warps 0-7  softmax, two threads to a query row (warps w and w + 4 share the rows 32 (w % 4) ..): both read the
//              row's 64 scores of a block for the maximum; each masks, exponentiates, sums and writes P (bf16,
//              swizzled) for its half of the keys; at the end each reads its half of O's columns, divides by
//              the row sum, stores.  Eight softmax warps a CTA, sixteen an SM: the kernel is bound by the
//              latencies inside a softmax warp (load, maximum, exponentials, store, barrier), not by a unit, so
//              what counts is how many such warps a scheduler can choose from
//   warp 8     TMA producer: Q once, then K and V blocks of 64 keys through the block table
//   warp 9     allocates tensor memory, issues the MMAs: S[j] = Q K_j^T, then O += P[j-1] V[j-1]
//
// O accumulates in tensor memory over all key blocks.  The exponentials of a row are taken against a
// reference maximum that is only raised when the row's running maximum has grown by more than 2^8
// since (p stays below 256, far inside bf16 and fp32 range); only then does the row's warp rescale its
// 32 lanes of O in tensor memory (load, multiply, store), after the previous PV has completed.  With
// causal prompts that happens in the first blocks of a row and hardly ever after.  S is double-
// buffered, so QK^T of block j+1 runs while block j is in softmax; P has one buffer, which the PV of
// block j has long left when the softmax of block j+1 wants to write it.  Shared memory (112 KB at
// head size 128), tensor memory (256 columns) and registers are sized so that two CTAs share an SM:
// the softmax of one hides the waits of the other.  Key blocks sit at absolute multiples of 64
// positions: a row's result depends on its own position and keys only.
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
constexpr int SOFTMAX_WARPS = 8;
constexpr int TC_ATT_THREADS = (SOFTMAX_WARPS + 2) * 32;
constexpr int KV_STAGES = 2;

struct PrefillTcArgs {
    const int* block_table;   // [B, max_blocks]
    const int* tiles;         // [n_tiles, 4]: first row, rows, first position, request index
    bf16* out;                // [T, nq * D]
    int* status;
    int nq, nkv, max_blocks, page_size, page_shift, mask_kind, mask_span;
    float scale_log2;
};

// Two fp32 operations in one instruction (sm_100 has packed f32x2 forms): the softmax warps are bound by the
// instructions they issue, so the scale-and-subtract and the row sum take pairs of columns at a time.
__device__ __forceinline__ uint64_t pack2(float lo, float hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "r"(__float_as_uint(lo)), "r"(__float_as_uint(hi)));
    return r;
}
__device__ __forceinline__ void unpack2(uint64_t v, float& lo, float& hi) {
    uint32_t a, b;
    asm("mov.b64 {%0, %1}, %2;" : "=r"(a), "=r"(b) : "l"(v));
    lo = __uint_as_float(a);
    hi = __uint_as_float(b);
}
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
    uint64_t d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}

enum { ERR_Q = 11, ERR_K = 12, ERR_V = 13, ERR_S = 14, ERR_P = 15, ERR_O = 16, ERR_EMPTY = 17, ERR_ALIGN = 18 };

template <int D>
struct AttCfg {
    static constexpr int HALVES = D / 64;
    static constexpr int Q_BYTES = TQ * D * 2;
    static constexpr int KV_BYTES = TK * D * 2;           // one K or V block
    static constexpr int P_BYTES = TQ * TK * 2;
    static constexpr int BAR_BYTES = 256;
    // the dynamic shared memory window has to start on a 1024-byte boundary (the kernel checks): there
    // is no room for padding when two CTAs of head size 128 share an SM
    static constexpr int SMEM = Q_BYTES + 2 * KV_STAGES * KV_BYTES + P_BYTES + BAR_BYTES;
    static constexpr int S_COL = 0;                        // S[2]: 64 columns each
    static constexpr int O_COL = 2 * TK;                   // O: D columns
    static constexpr int TMEM_COLS = 256;                  // 128 + D <= 256
};

template <int D>
__global__ void __launch_bounds__(TC_ATT_THREADS, 2)
attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap q_map, const __grid_constant__ CUtensorMap kv_map,
                       const PrefillTcArgs a) {
    using Cfg = AttCfg<D>;
    extern __shared__ __align__(1024) uint8_t smem[];
    if (smem_u32(smem) & 1023u) {                  // the swizzled tiles need it; nothing has been set up yet
        if (threadIdx.x == 0) atomicExch(a.status, ERR_ALIGN);
        return;
    }
    uint8_t* q_s = smem;
    uint8_t* k_s = q_s + Cfg::Q_BYTES;                          // [stages][halves][64 keys][64]
    uint8_t* v_s = k_s + KV_STAGES * Cfg::KV_BYTES;
    uint8_t* p_s = v_s + KV_STAGES * Cfg::KV_BYTES;             // [128 rows][64 keys]
    uint64_t* bars = reinterpret_cast<uint64_t*>(p_s + Cfg::P_BYTES);
    uint64_t* q_full = bars;
    uint64_t* k_full = bars + 1;
    uint64_t* k_empty = k_full + KV_STAGES;
    uint64_t* v_full = k_empty + KV_STAGES;
    uint64_t* v_empty = v_full + KV_STAGES;
    uint64_t* s_full = v_empty + KV_STAGES;       // [2]
    uint64_t* p_full = s_full + 2;                // 128 arrivals, once per block
    uint64_t* pv_done = p_full + 1;               // completes once per block, when its PV is done
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(pv_done + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // The last tiles of a prompt have the most keys: start them first, for every head (the head is the fast
    // index of the grid, so CTAs are handed out tile by tile, all heads of a tile together: the short tiles
    // of all heads fill the tail, and the query heads of a kv head read its keys at the same time).
    const int* tile = a.tiles + (size_t)(gridDim.y - 1 - blockIdx.y) * 4;
    const int row0 = tile[0], n_rows = tile[1], p0 = tile[2];
    const int* table = a.block_table + (size_t)tile[3] * a.max_blocks;
    const int head = blockIdx.x;
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
        mbar_init(&s_full[0], 1); mbar_init(&s_full[1], 1);
        mbar_init(p_full, SOFTMAX_WARPS * 32);
        mbar_init(pv_done, 1);
        fence_barrier_init();
    }
    if (warp == SOFTMAX_WARPS + 1) {
        tmem_alloc(tmem_slot, Cfg::TMEM_COLS);
        tmem_relinquish();
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == SOFTMAX_WARPS) {
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
    } else if (warp == SOFTMAX_WARPS + 1) {
        // ---- MMA issuer ------------------------------------------------------------------------
        if (lane == 0) {
            const uint32_t idesc_qk = instr_desc_bf16(TQ, TK);
            const uint32_t idesc_pv = instr_desc_bf16(TQ, D, true);
            bool ok = mbar_wait(q_full, 0);
            if (!ok) atomicExch(a.status, ERR_Q);
            auto pv = [&](int i) -> bool {
                const int st = i % KV_STAGES;
                if (!mbar_wait(p_full, i & 1)) { atomicExch(a.status, ERR_P); return false; }
                if (!mbar_wait(&v_full[st], (i / KV_STAGES) & 1)) { atomicExch(a.status, ERR_V); return false; }
                tcgen05_fence_after();
                const uint8_t* pt = p_s;
                const uint8_t* vt = v_s + st * Cfg::KV_BYTES;
#pragma unroll
                for (int ks = 0; ks < TK / 16; ++ks)
                    mma_bf16_ss(tmem_base + Cfg::O_COL, smem_desc_k_sw128(pt, ks * 32),
                                smem_desc_mn_sw128(vt, TK * 128, ks * 2048), idesc_pv, (i | ks) != 0);
                mma_commit(&v_empty[st]);
                mma_commit(pv_done);
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
        // ---- softmax: two threads to a query row ---------------------------------------------------
        constexpr int HALF = TK / 2;                         // keys of a block per thread
        const int quarter = warp & 3, half = warp >> 2;
        const int r = quarter * 32 + lane;
        const int pos_r = p0 + r;
        const int lo_r = visible_lo(pos_r, a.mask_kind, a.mask_span);
        const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
        constexpr float RAISE = 8.0f;       // in log2 units: the reference maximum lags by at most this much
        const float scale = a.scale_log2;   // > 0: the maximum of the raw scores is the maximum of the scaled ones
        float m_ref = -INFINITY, l_run = 0.0f;      // m_ref in log2 units; l_run: this thread's half of the row sum
        bool ok = true;

        for (int j = 0; j < n_blocks; ++j) {
            const int b = j & 1;
            if (!mbar_wait(&s_full[b], (j >> 1) & 1)) { atomicExch(a.status, ERR_S); ok = false; break; }
            tcgen05_fence_after();
            const int key0 = (kb_first + j) * TK;
            const bool hidden = !(key0 + TK - 1 <= pos_r && key0 >= lo_r);   // some keys of the block are hidden from this row
            // the other half's scores first, for the maximum alone; then this thread's own, which it keeps
            uint32_t sv[HALF];
            tmem_ld_32_nowait(lane_addr + Cfg::S_COL + b * TK + (1 - half) * HALF, sv);
            tmem_ld_wait();
            if (hidden) {
#pragma unroll
                for (int c = 0; c < HALF; ++c) {
                    const int key = key0 + (1 - half) * HALF + c;
                    if (!(key <= pos_r && key >= lo_r)) sv[c] = 0xff800000u;    // -inf
                }
            }
            float m0 = fmax3(__uint_as_float(sv[0]), __uint_as_float(sv[1]), __uint_as_float(sv[2]));
            float m1 = fmax3(__uint_as_float(sv[3]), __uint_as_float(sv[4]), __uint_as_float(sv[5]));
#pragma unroll
            for (int c = 6; c + 3 < HALF; c += 4) {
                m0 = fmax3(m0, __uint_as_float(sv[c]), __uint_as_float(sv[c + 1]));
                m1 = fmax3(m1, __uint_as_float(sv[c + 2]), __uint_as_float(sv[c + 3]));
            }
            const float m_other = fmax3(m0, m1, fmaxf(__uint_as_float(sv[HALF - 2]), __uint_as_float(sv[HALF - 1])));
            auto load_own = [&]() {
                tmem_ld_32_nowait(lane_addr + Cfg::S_COL + b * TK + half * HALF, sv);
                tmem_ld_wait();
                if (hidden) {
#pragma unroll
                    for (int c = 0; c < HALF; ++c) {
                        const int key = key0 + half * HALF + c;
                        if (!(key <= pos_r && key >= lo_r)) sv[c] = 0xff800000u;    // -inf: its exponential is 0
                    }
                }
            };
            load_own();
            m0 = fmax3(__uint_as_float(sv[0]), __uint_as_float(sv[1]), __uint_as_float(sv[2]));
            m1 = fmax3(__uint_as_float(sv[3]), __uint_as_float(sv[4]), __uint_as_float(sv[5]));
#pragma unroll
            for (int c = 6; c + 3 < HALF; c += 4) {
                m0 = fmax3(m0, __uint_as_float(sv[c]), __uint_as_float(sv[c + 1]));
                m1 = fmax3(m1, __uint_as_float(sv[c + 2]), __uint_as_float(sv[c + 3]));
            }
            const float m_mine = fmax3(m0, m1, fmaxf(__uint_as_float(sv[HALF - 2]), __uint_as_float(sv[HALF - 1])));
            const float m_blk = fmaxf(m_mine, m_other) * scale;      // the same number in both threads of the row
            // raise the reference maximum only when this block's maximum is far above it; the rows of a warp
            // share the decision to touch O (and the row's two warps decide alike), each row uses its own factor
            const bool raise = m_blk > m_ref + RAISE;               // also true for the row's first visible block
            if (__any_sync(0xffffffffu, raise)) {
                const float m_new = fmaxf(m_ref, m_blk);
                const float factor = (m_ref == -INFINITY) ? 0.0f : exp2f(m_ref - m_new);   // nothing of value in O yet
                if (j > 0) {
                    // O holds the sums of blocks 0 .. j-1 once the PV of block j-1 is complete; this thread
                    // rescales its half of the row's columns
                    if (!mbar_wait(pv_done, (j - 1) & 1)) { atomicExch(a.status, ERR_O); ok = false; break; }
                    tcgen05_fence_after();
#pragma unroll
                    for (int c0 = half * (D / 2); c0 < (half + 1) * (D / 2); c0 += 32) {
                        uint32_t v[32];
                        tmem_ld_32_nowait(lane_addr + Cfg::O_COL + c0, v);
                        tmem_ld_wait();
#pragma unroll
                        for (int i2 = 0; i2 < 32; ++i2) v[i2] = __float_as_uint(__uint_as_float(v[i2]) * factor);
                        tmem_st_32(lane_addr + Cfg::O_COL + c0, v);
                    }
                    tmem_st_wait();
                    load_own();          // the scores again: they need not live in registers across the rescaling
                }
                l_run *= factor;
                m_ref = m_new;
            }
            // exp2(s * scale - m_ref): one fused multiply-add and one ex2 per score; a hidden score is -inf and
            // gives 0, also for a row that has seen no key yet (its reference stands in as 0)
            const float neg_m = (m_ref == -INFINITY) ? 0.0f : -m_ref;
            uint32_t packed[HALF / 2];
            const uint64_t scale2 = pack2(scale, scale), neg_m2 = pack2(neg_m, neg_m);
            uint64_t l2 = pack2(0.0f, 0.0f);
#pragma unroll
            for (int c = 0; c < HALF; c += 2) {
                float x0, x1;
                unpack2(fma2(pack2(__uint_as_float(sv[c]), __uint_as_float(sv[c + 1])), scale2, neg_m2), x0, x1);
                const float e0 = ex2_approx(x0), e1 = ex2_approx(x1);
                l2 = add2(l2, pack2(e0, e1));
                __nv_bfloat162 pr = __floats2bfloat162_rn(e0, e1);
                packed[c / 2] = *reinterpret_cast<uint32_t*>(&pr);
            }
            float l0, l1;
            unpack2(l2, l0, l1);
            l_run += l0 + l1;
            // P may be overwritten once the MMAs that read the previous block's are done
            if (j >= 1 && !mbar_wait(pv_done, (j - 1) & 1)) { atomicExch(a.status, ERR_P); ok = false; break; }
            uint8_t* prow = p_s + r * 128;
#pragma unroll
            for (int ch = 0; ch < 4; ++ch)
                *reinterpret_cast<uint4*>(prow + (((half * 4 + ch) ^ (r & 7)) << 4)) =
                    make_uint4(packed[ch * 4], packed[ch * 4 + 1], packed[ch * 4 + 2], packed[ch * 4 + 3]);
            fence_proxy_async();
            tcgen05_fence_before();
            mbar_arrive(p_full);
        }
        if (ok && !mbar_wait(pv_done, (n_blocks - 1) & 1)) { atomicExch(a.status, ERR_O); ok = false; }
        // the row sum: the two halves meet in the P buffer, which nothing reads any more (every softmax thread
        // comes here, whatever its waits said, so the barrier is complete)
        float* l_s = reinterpret_cast<float*>(p_s);
        l_s[half * TQ + r] = l_run;
        named_barrier_all(1, SOFTMAX_WARPS * 32, true);
        const float l_row = l_s[r] + l_s[TQ + r];          // the same order in both threads
        if (ok) {
            tcgen05_fence_after();
            const float inv = 1.0f / l_row;
            bf16* dst = a.out + ((size_t)(row0 + r) * a.nq + head) * D;
#pragma unroll
            for (int c0 = half * (D / 2); c0 < (half + 1) * (D / 2); c0 += 32) {
                uint32_t v[32];
                tmem_ld_32_nowait(lane_addr + Cfg::O_COL + c0, v);      // whole-warp operation: all rows take part
                tmem_ld_wait();
                if (r < n_rows) {
#pragma unroll
                    for (int c = 0; c < 32; c += 8) {
                        uint4 w;
                        __nv_bfloat162 h0 = __floats2bfloat162_rn(__uint_as_float(v[c]) * inv, __uint_as_float(v[c + 1]) * inv);
                        __nv_bfloat162 h1 = __floats2bfloat162_rn(__uint_as_float(v[c + 2]) * inv, __uint_as_float(v[c + 3]) * inv);
                        __nv_bfloat162 h2 = __floats2bfloat162_rn(__uint_as_float(v[c + 4]) * inv, __uint_as_float(v[c + 5]) * inv);
                        __nv_bfloat162 h3 = __floats2bfloat162_rn(__uint_as_float(v[c + 6]) * inv, __uint_as_float(v[c + 7]) * inv);
                        w.x = *reinterpret_cast<uint32_t*>(&h0); w.y = *reinterpret_cast<uint32_t*>(&h1);
                        w.z = *reinterpret_cast<uint32_t*>(&h2); w.w = *reinterpret_cast<uint32_t*>(&h3);
                        *reinterpret_cast<uint4*>(dst + c0 + c) = w;
                    }
                }
            }
        }
    }
    tcgen05_fence_before();
    __syncthreads();
    if (warp == SOFTMAX_WARPS + 1) {
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
    attn_prefill_tc_kernel<D><<<dim3(a.nq, n_tiles), TC_ATT_THREADS, Cfg::SMEM, stream>>>(qm, kvm, a);
    SHARPI_CHECK_LAUNCH();
    return SHARPI_OK;
}

// q [T, nq, d] bf16; kv [num_pages, 2, nkv, page_size, d] bf16; tiles of up to 128 rows.
SHARPI_API int sharpi_attention_prefill_tc(const void* q, const void* kv, const int* block_table, const int* tiles,
                                           void* out, int* status, int T, int num_pages, int n_tiles, int nq, int nkv,
                                           int d, int max_blocks, int page_size, int mask_kind, int mask_span,
                                           float scale, cudaStream_t stream) {
    if (n_tiles <= 0) return SHARPI_OK;
    if (n_tiles > 65535) return SHARPI_BAD_ARGUMENT;        // tiles are the grid's second extent
    if (nq <= 0 || nkv <= 0 || nq % nkv != 0 || max_blocks <= 0 || nq > 65535 || !status) return SHARPI_BAD_ARGUMENT;
    if (d != 64 && d != 128) return SHARPI_BAD_ARGUMENT;
    if (!(scale > 0.0f)) return SHARPI_BAD_ARGUMENT;
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
