// Paged attention for rows that bring one query each (decode), bf16 cache, split over the keys.
//
// The work is reading every visible key and value once, so the kernel is organised around
// bytes in flight: one CTA takes one (row, kv head, split of 256 keys) and serves all the query
// heads of that kv head at once, so keys and values are read once per group, not once per
// query head.  For rows of unequal lengths the grid's first extent counts the splits of all rows together
// (a CTA finds its row by a prefix sum over the rows' split counts), so a batch of one long row and many
// short ones launches what it has, not rows times the longest row's splits.  Splits sit at absolute multiples of 256 positions, so the order in which a row's
// keys are reduced depends on the row's position alone, never on the batch.  Each CTA writes an
// unnormalised partial (max, sum, weighted values); a second kernel merges a row's partials.
//
// The reference's counterparts: llm_attention_splitkv_grouped + llm_attention_combine (fixed
// 512-key splits, one block per (kv head, split), scalar math;
// src/SharpInference.Cuda/CudaTextKernels.cs:8829-9072) and llm_attention_ragged for several
// sequences in one launch (src/SharpInference.Cuda/CudaRaggedKernels.cs:291-325).  Here QK^T and PV
// run on the tensor cores (m16n8k16, the query heads of a group padded to 16 rows), softmax
// statistics are fp32, masks are full / chunk / window as in common.cuh.
#include "common.cuh"
#include "mma_sync.cuh"
#include "sm100.cuh"
#include "tensor_map.cuh"
#include <string.h>

using namespace mma16;

constexpr int DEC_SPLIT = 256;   // keys per CTA
constexpr int DEC_CHUNK = 16;    // keys per warp pass; a warp owns 64 keys of the split and double-buffers its passes
constexpr int DEC_WARPS = 4;
constexpr int DEC_THREADS = DEC_WARPS * 32;
constexpr int DEC_WARP_KEYS = DEC_SPLIT / DEC_WARPS;

struct DecodeArgs {
    const bf16* q;            // [T, nq, D]
    const bf16* kv;           // [pages, 2, nkv, page_size, D]
    const int* block_table;   // [B, max_blocks]
    const int* row_req;       // [T]
    const int* positions;     // [T]
    const int* rows;          // [R] rows served by this launch, or null for rows 0 .. R-1
    float* part_o;            // [R, nq, max_splits, D]
    float* part_ml;           // [R, nq, max_splits, 2]   (max in log2 units, sum)
    bf16* out;                // [T, nq * D]
    int nq, nkv, max_blocks, page_size, page_shift, mask_kind, mask_span, max_splits;
    int num_rows;             // R
    float scale_log2;         // softmax scale * log2(e)
    int* status;              // device word for a wait that gave up (TMA path)
};

template <int D>
__device__ __forceinline__ void decode_load_chunk(const DecodeArgs& a, const int* table, int kvh, size_t plane,
                                                  int chunk0, int k_begin, int k_end, bf16* k_s, bf16* v_s, int lane) {
    constexpr int LD = D + 8, VEC = D / 8;
#pragma unroll
    for (int idx = lane; idx < DEC_CHUNK * VEC; idx += 32) {
        const int row = idx / VEC, col = idx % VEC;
        const int key = chunk0 + row;
        bool valid = key >= k_begin && key <= k_end;
        int page = -1, off = 0;
        if (valid) {
            const int blk = a.page_shift >= 0 ? (key >> a.page_shift) : (key / a.page_size);
            off = key - blk * a.page_size;
            page = table[blk];
        }
        valid = valid && page >= 0;
        const bf16* src = a.kv;
        if (valid) src = a.kv + (size_t)page * 2 * plane + ((size_t)kvh * a.page_size + off) * D + col * 8;
        cp_async_16(k_s + row * LD + col * 8, src, valid ? 16 : 0);
        cp_async_16(v_s + row * LD + col * 8, valid ? src + plane : src, valid ? 16 : 0);
    }
}

// Two ways of bringing a pass's 16 keys and values into shared memory:
//   TMA == false  cp.async, 16 bytes per thread, rows padded by 8 elements against bank conflicts; any
//                 page size, any head size that is a multiple of 16.
//   TMA == true   one thread of the warp issues bulk tensor copies (a [16 rows x 64 elements] box per half
//                 of the head size, 128-byte swizzle) that complete on an mbarrier; ldmatrix undoes the
//                 swizzle in its addresses.  Needs pages of a multiple of 16 positions and a head size of
//                 64 or 128, and cuts the instructions spent on loading to a few per pass.
template <int D, bool TMA, bool COMPACT>
__global__ void __launch_bounds__(DEC_THREADS, 3) attn_decode_split_kernel(const __grid_constant__ CUtensorMap kv_map,
                                                                           DecodeArgs a) {
    constexpr int LD = TMA ? 64 : D + 8;   // row pitch in elements: swizzled 128-byte rows, or padded rows
    constexpr int VEC = D / 8;             // 16-byte pieces per row
    constexpr int HALVES = TMA ? D / 64 : 1;
    constexpr int BUF = 2 * DEC_CHUNK * (TMA ? D : D + 8);     // one buffer: K rows then V rows, in elements
    constexpr int QLD = D + 8;
    extern __shared__ __align__(1024) uint8_t smem_bytes[];
    // TMA: the staging buffers come first so that they sit on 1024-byte boundaries (each is a multiple of 1024)
    bf16* kv_s = reinterpret_cast<bf16*>(smem_bytes);                       // [warps][2 buffers][K|V][...]
    bf16* q_s = kv_s + DEC_WARPS * 2 * BUF;                                  // [16][QLD]
    uint64_t* bars = reinterpret_cast<uint64_t*>(q_s + 16 * QLD);            // [warps][2]

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    pdl_wait();
    const int G = a.nq / a.nkv;
    const int groups = (G + 15) / 16;
    const int kvh = blockIdx.y / groups, hg = blockIdx.y % groups;
    const int head0 = kvh * G + hg * 16;
    const int heads_here = min(16, G - hg * 16);
    // COMPACT: blockIdx.x counts splits over all rows: find the row whose splits hold it (every warp does the
    // same scan over the rows, 32 at a time) and the split's number within that row.  Otherwise the grid is
    // (splits of the longest row, ., rows), which costs nothing to decode and suits rows of similar lengths.
    int ri = -1, r = 0, pos = 0, lo = 0, split_in_row = 0;
    if (!COMPACT) {
        ri = blockIdx.z;
        r = a.rows ? a.rows[ri] : ri;
        pos = a.positions[r];
        lo = visible_lo(pos, a.mask_kind, a.mask_span);
        split_in_row = blockIdx.x;
    } else {
        const int item = blockIdx.x;
        int base = 0;
        for (int r0 = 0; r0 < a.num_rows; r0 += 32) {
            const int i = r0 + lane;
            int rr = 0, p = 0, l = 0, n = 0;
            if (i < a.num_rows) {
                rr = a.rows ? a.rows[i] : i;
                p = a.positions[rr];
                l = visible_lo(p, a.mask_kind, a.mask_span);
                n = p / DEC_SPLIT - l / DEC_SPLIT + 1;
            }
            int incl = n;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int v = __shfl_up_sync(0xffffffffu, incl, o);
                if (lane >= o) incl += v;
            }
            const int here = __shfl_sync(0xffffffffu, incl, 31);
            if (item < base + here) {
                const int owner = __ffs(__ballot_sync(0xffffffffu, item < base + incl)) - 1;
                ri = r0 + owner;
                r = __shfl_sync(0xffffffffu, rr, owner);
                pos = __shfl_sync(0xffffffffu, p, owner);
                lo = __shfl_sync(0xffffffffu, l, owner);
                split_in_row = item - base - __shfl_sync(0xffffffffu, incl - n, owner);
                break;
            }
            base += here;
        }
    }
    if (ri < 0) return;          // past the last row's last split (pdl_wait has been called above)
    const int split = lo / DEC_SPLIT + split_in_row;
    const int k_begin = max(lo, split * DEC_SPLIT);
    const int k_end = min(pos, split * DEC_SPLIT + DEC_SPLIT - 1);
    if (k_begin > k_end) return;

    bf16* w_s = kv_s + (size_t)warp * 2 * BUF;
    const int* table = a.block_table + (size_t)a.row_req[r] * a.max_blocks;
    const size_t plane = (size_t)a.nkv * a.page_size * D;

    // this warp's keys and its first pass are requested before anything else
    const int wbase = split * DEC_SPLIT + warp * DEC_WARP_KEYS;
    const int wk0 = max(k_begin, wbase), wk1 = min(k_end, wbase + DEC_WARP_KEYS - 1);
    const int c_first = (wk0 - wbase) / DEC_CHUNK, c_last = (wk1 - wbase) / DEC_CHUNK;    // meaningful if wk0 <= wk1
    const bool has_keys = wk0 <= wk1;
    uint64_t* my_bars = bars + warp * 2;
    uint32_t phase[2] = {0, 0};
    bool tma_ok = true;

    // One pass by TMA: K and V of 16 consecutive keys of one page (a pass never straddles pages, which
    // hold a multiple of 16 positions), as 2 * HALVES boxes of [16 rows x 64 elements].
    auto tma_issue = [&](int chunk0, int buf) {
        const int blk = chunk0 >> a.page_shift;
        const int page = table[blk];
        const int off = chunk0 - (blk << a.page_shift);
        bf16* dst = w_s + buf * BUF;
        const int row_k = ((page * 2 + 0) * a.nkv + kvh) * a.page_size + off;
        const int row_v = ((page * 2 + 1) * a.nkv + kvh) * a.page_size + off;
        sm100::mbar_arrive_expect_tx(&my_bars[buf], 2 * DEC_CHUNK * D * 2);
#pragma unroll
        for (int hf = 0; hf < HALVES; ++hf) {
            sm100::tma_load_2d(dst + hf * DEC_CHUNK * 64, &kv_map, &my_bars[buf], hf * 64, row_k);
            sm100::tma_load_2d(dst + DEC_CHUNK * D + hf * DEC_CHUNK * 64, &kv_map, &my_bars[buf], hf * 64, row_v);
        }
    };
    if (TMA && (sm100::smem_u32(kv_s) & 1023u) != 0) {
        // the swizzle that ldmatrix undoes assumes staging buffers on 1024-byte boundaries
        if (threadIdx.x == 0) atomicExch(a.status, 5);
        return;
    }
    if (TMA) {
        if (lane == 0) {
            sm100::mbar_init(&my_bars[0], 1);
            sm100::mbar_init(&my_bars[1], 1);
            sm100::fence_barrier_init();
        }
        __syncwarp();
        if (has_keys && lane == 0) tma_issue(wbase + c_first * DEC_CHUNK, 0);
    } else if (has_keys) {
        decode_load_chunk<D>(a, table, kvh, plane, wbase + c_first * DEC_CHUNK, k_begin, k_end, w_s, w_s + DEC_CHUNK * LD, lane);
        cp_async_commit();
    }

    // queries of this group: rows >= heads_here are zero
    for (int idx = threadIdx.x; idx < 16 * VEC; idx += DEC_THREADS) {
        const int g = idx / VEC, c = idx % VEC;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (g < heads_here) v = *reinterpret_cast<const uint4*>(a.q + ((size_t)r * a.nq + head0 + g) * D + c * 8);
        *reinterpret_cast<uint4*>(q_s + g * QLD + c * 8) = v;
    }
    __syncthreads();
    uint32_t qa[D / 16][4];
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) ldmatrix_x4(qa[ks], q_s + (lane % 16) * QLD + ks * 16 + (lane / 16) * 8);

    // Address of the 8-element piece at (row, first column col) of a staged K or V tile.  With TMA the
    // tile is [halves][16 rows][64 elements] and the 16-byte pieces of a row are XOR-swizzled by row % 8.
    auto piece = [&](bf16* tile, int row, int col) -> bf16* {
        if (TMA) return tile + (col >> 6) * (DEC_CHUNK * 64) + row * 64 + ((((col & 63) >> 3) ^ (row & 7)) << 3);
        return tile + row * LD + col;
    };

    float o[D / 8][4];
#pragma unroll
    for (int i = 0; i < D / 8; ++i)
#pragma unroll
        for (int e = 0; e < 4; ++e) o[i][e] = 0.0f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.0f, 0.0f};

    if (has_keys) {
        for (int c = c_first; c <= c_last; ++c) {
            const int buf = (c - c_first) & 1;
            bf16* k_s = w_s + buf * BUF;
            bf16* v_s = k_s + (TMA ? DEC_CHUNK * D : DEC_CHUNK * LD);
            if (TMA) {
                if (c < c_last && lane == 0) tma_issue(wbase + (c + 1) * DEC_CHUNK, buf ^ 1);
                const bool landed = sm100::mbar_wait(&my_bars[buf], phase[buf]);
                if (!__all_sync(0xffffffffu, landed)) {     // the whole warp leaves together
                    tma_ok = false;
                    break;
                }
                phase[buf] ^= 1;
            } else if (c < c_last) {       // ask for the next pass while this one is computed
                bf16* nk = w_s + (buf ^ 1) * BUF;
                decode_load_chunk<D>(a, table, kvh, plane, wbase + (c + 1) * DEC_CHUNK, k_begin, k_end, nk, nk + DEC_CHUNK * LD, lane);
                cp_async_commit();
                cp_async_wait<1>();
            } else {
                cp_async_wait<0>();
            }
            __syncwarp();
            const int chunk0 = wbase + c * DEC_CHUNK;

            // S = Q K^T for 16 keys: 2 tiles of 8 keys
            float s[2][4];
#pragma unroll
            for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
                for (int e = 0; e < 4; ++e) s[nt][e] = 0.0f;
#pragma unroll
                for (int k2 = 0; k2 < D / 32; ++k2) {
                    uint32_t b[4];
                    ldmatrix_x4(b, piece(k_s, nt * 8 + (lane % 8), k2 * 32 + (lane / 8) * 8));
                    mma_bf16(s[nt], qa[2 * k2], b[0], b[1]);
                    mma_bf16(s[nt], qa[2 * k2 + 1], b[2], b[3]);
                }
                if (D % 32 != 0) {
                    uint32_t b[2];
                    ldmatrix_x2(b, piece(k_s, nt * 8 + (lane % 8), (D - 16) + ((lane / 8) % 2) * 8));
                    mma_bf16(s[nt], qa[D / 16 - 1], b[0], b[1]);
                }
            }
            // mask, running max and sum (rows lane/4 and lane/4 + 8 of the group)
            float m_c[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int key = chunk0 + nt * 8 + (lane % 4) * 2 + (e & 1);
                    const bool valid = key >= k_begin && key <= k_end;
                    s[nt][e] = valid ? s[nt][e] * a.scale_log2 : -INFINITY;
                    m_c[e >> 1] = fmaxf(m_c[e >> 1], s[nt][e]);
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
            for (int nt = 0; nt < 2; ++nt)
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
            // O += P V: P (16 x 16) straight from the S accumulators
            uint32_t pa[4];
            pa[0] = pack_bf16(s[0][0], s[0][1]);
            pa[1] = pack_bf16(s[0][2], s[0][3]);
            pa[2] = pack_bf16(s[1][0], s[1][1]);
            pa[3] = pack_bf16(s[1][2], s[1][3]);
#pragma unroll
            for (int d2 = 0; d2 < D / 16; ++d2) {
                uint32_t b[4];
                ldmatrix_x4_trans(b, piece(v_s, (lane % 8) + ((lane / 8) % 2) * 8, d2 * 16 + (lane / 16) * 8));
                mma_bf16(o[2 * d2], pa, b[0], b[1]);
                mma_bf16(o[2 * d2 + 1], pa, b[2], b[3]);
            }
            __syncwarp();
        }
    }
    if (TMA && !tma_ok) {
        // a copy did not complete in time: record it, give a copy that may still be in flight time to land
        if (lane == 0) atomicExch(a.status, 4);
        sm100::mbar_wait(&my_bars[0], phase[0], 1u << 14);
        sm100::mbar_wait(&my_bars[1], phase[1], 1u << 14);
        m_run[0] = m_run[1] = -INFINITY;
        l_run[0] = l_run[1] = 0.0f;
    }

    // each warp leaves its partial in its own staging area, then the block merges the four
    float* o_w = reinterpret_cast<float*>(w_s);                 // [16][D] (every copy into the buffers has landed)
    float* ml_w = o_w + 16 * D;                                  // [16][2]
#pragma unroll
    for (int i = 0; i < D / 8; ++i)
#pragma unroll
        for (int e = 0; e < 4; ++e)
            o_w[(lane / 4 + 8 * (e >> 1)) * D + i * 8 + (lane % 4) * 2 + (e & 1)] = o[i][e];
    if (lane % 4 == 0) {
        ml_w[(lane / 4) * 2] = m_run[0];
        ml_w[(lane / 4) * 2 + 1] = l_run[0];
        ml_w[(lane / 4 + 8) * 2] = m_run[1];
        ml_w[(lane / 4 + 8) * 2 + 1] = l_run[1];
    }
    __syncthreads();
    constexpr size_t warp_stride = (size_t)2 * BUF * sizeof(bf16) / sizeof(float);
    const float* base_o = reinterpret_cast<const float*>(kv_s);
    for (int idx = threadIdx.x; idx < heads_here * D; idx += DEC_THREADS) {
        const int g = idx / D, dd = idx % D;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < DEC_WARPS; ++w) M = fmaxf(M, base_o[w * warp_stride + 16 * D + g * 2]);
        float acc = 0.0f, L = 0.0f;
#pragma unroll
        for (int w = 0; w < DEC_WARPS; ++w) {
            const float mw = base_o[w * warp_stride + 16 * D + g * 2];
            const float f = (mw == -INFINITY) ? 0.0f : exp2f(mw - M);
            acc += f * base_o[w * warp_stride + g * D + dd];
            L += f * base_o[w * warp_stride + 16 * D + g * 2 + 1];
        }
        const size_t slot = ((size_t)ri * a.nq + head0 + g) * a.max_splits + split_in_row;
        a.part_o[slot * D + dd] = acc;
        if (dd == 0) {
            a.part_ml[slot * 2] = M;
            a.part_ml[slot * 2 + 1] = L;
        }
    }
}

// One block per (row, query head): the row's partials, weighted by exp2(max_s - max) and normalised.  A warp
// takes one split at a time (its D floats are one coalesced read, four per lane) and every n-th (n warps a block)
// split after it, several loads in flight; the warps' sums are then added in warp order, so the result
// depends on the row's position alone.
constexpr int MERGE_WARPS = 32;          // at most; the launch takes half of them for rows of few splits
constexpr int MERGE_THREADS = MERGE_WARPS * 32;
constexpr int MERGE_UNROLL = 4;
constexpr int MERGE_WIDE_FROM = 256;     // splits from which a block of MERGE_WARPS warps pays

template <int D>
__global__ void __launch_bounds__(MERGE_THREADS) attn_decode_merge_kernel(DecodeArgs a) {
    static_assert(D % 4 == 0 && D <= 128, "a warp reads a split's D floats four per lane");
    __shared__ float4 acc_s[MERGE_WARPS][D / 4];
    __shared__ float l_s[MERGE_WARPS];
    __shared__ float scratch[32];
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int ri = blockIdx.x, head = blockIdx.y;
    const int r = a.rows ? a.rows[ri] : ri;
    const int pos = a.positions[r];
    const int lo = visible_lo(pos, a.mask_kind, a.mask_span);
    const int n_s = pos / DEC_SPLIT - lo / DEC_SPLIT + 1;
    // how many warps share a row is a matter of the row alone (the block may have more), as the order of the sum
    const int warps = n_s >= MERGE_WIDE_FROM ? MERGE_WARPS : MERGE_WARPS / 2;
    const size_t slot0 = ((size_t)ri * a.nq + head) * a.max_splits;
    const float2* ml = reinterpret_cast<const float2*>(a.part_ml) + slot0;
    float m = -INFINITY;
    for (int s = threadIdx.x; s < n_s; s += blockDim.x) m = fmaxf(m, ml[s].x);
    const float M = block_max(m, scratch);
    const bool active = lane < D / 4;
    const float4* po = reinterpret_cast<const float4*>(a.part_o + slot0 * D) + (active ? lane : 0);
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    float l = 0.0f;
    for (int s0 = warp; s0 < n_s && warp < warps; s0 += warps * MERGE_UNROLL) {
        float2 st[MERGE_UNROLL];
        float4 v[MERGE_UNROLL];
#pragma unroll
        for (int u = 0; u < MERGE_UNROLL; ++u) {
            const int s = s0 + u * warps;
            const bool ok = s < n_s;
            st[u] = ok ? ml[s] : make_float2(-INFINITY, 0.0f);
            v[u] = ok ? po[(size_t)s * (D / 4)] : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int u = 0; u < MERGE_UNROLL; ++u) {
            const float w = exp2f(st[u].x - M);       // 0 for the splits past the end
            l += w * st[u].y;
            acc.x += w * v[u].x; acc.y += w * v[u].y; acc.z += w * v[u].z; acc.w += w * v[u].w;
        }
    }
    if (active && warp < warps) acc_s[warp][lane] = acc;
    if (lane == 0 && warp < warps) l_s[warp] = l;
    __syncthreads();
    if (threadIdx.x < D / 4) {
        float4 o = acc_s[0][threadIdx.x];
        float L = l_s[0];
        for (int w = 1; w < warps; ++w) {
            const float4 t = acc_s[w][threadIdx.x];
            o.x += t.x; o.y += t.y; o.z += t.z; o.w += t.w;
            L += l_s[w];
        }
        const float inv = 1.0f / L;
        bf16* dst = a.out + ((size_t)r * a.nq + head) * D + threadIdx.x * 4;
        __nv_bfloat162 p0 = __floats2bfloat162_rn(o.x * inv, o.y * inv), p1 = __floats2bfloat162_rn(o.z * inv, o.w * inv);
        uint2 pk;
        pk.x = *reinterpret_cast<uint32_t*>(&p0);
        pk.y = *reinterpret_cast<uint32_t*>(&p1);
        *reinterpret_cast<uint2*>(dst) = pk;
    }
}

// A grid over all rows' splits together pays when rows times the longest row's splits would leave a fifth of
// the CTAs without work; otherwise the grid is (splits, kv heads, rows).
template <int D, bool TMA, bool COMPACT>
static int launch_split(const CUtensorMap& map, const DecodeArgs& a, int R, int splits, int items, cudaStream_t stream) {
    constexpr int ROW = TMA ? D : D + 8;
    constexpr int SMEM = (DEC_WARPS * 2 * 2 * DEC_CHUNK * ROW + 16 * (D + 8)) * 2 + DEC_WARPS * 2 * 8;
    static_assert(2 * 2 * DEC_CHUNK * ROW * 2 >= (16 * D + 32) * 4, "a warp's staging area must hold its partial");
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(attn_decode_split_kernel<D, TMA, COMPACT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 SMEM) != cudaSuccess)
            return SHARPI_LAUNCH_FAILED;
        configured = true;
    }
    const int G = a.nq / a.nkv;
    const dim3 grid = COMPACT ? dim3(items, a.nkv * ((G + 15) / 16)) : dim3(splits, a.nkv * ((G + 15) / 16), R);
    auto kern = attn_decode_split_kernel<D, TMA, COMPACT>;
    SHARPI_LAUNCH_PDL(kern, grid, DEC_THREADS, SMEM, stream, map, a);
    return SHARPI_OK;
}

template <int D, bool TMA>
static int launch_split(const CUtensorMap& map, const DecodeArgs& a, int R, int splits, int items, cudaStream_t stream) {
    if ((long long)items * 5 < (long long)R * splits * 4) return launch_split<D, TMA, true>(map, a, R, splits, items, stream);
    return launch_split<D, TMA, false>(map, a, R, splits, items, stream);
}

template <int D>
static int launch_decode(const DecodeArgs& a, int R, int splits, int items, long long pool_rows, cudaStream_t stream) {
    CUtensorMap map;
    memset(&map, 0, sizeof(map));
    int rc;
    const bool tma = (D % 64 == 0) && a.page_shift >= 4 && a.status != nullptr && pool_rows > 0;
    if (tma) {
        if (!tmap::make_bf16_map(&map, a.kv, (uint64_t)D, (uint64_t)pool_rows, 0, 64, DEC_CHUNK)) return SHARPI_LAUNCH_FAILED;
        rc = launch_split<D, (D % 64 == 0)>(map, a, R, splits, items, stream);
    } else {
        rc = launch_split<D, false>(map, a, R, splits, items, stream);
    }
    if (rc != SHARPI_OK) return rc;
    SHARPI_LAUNCH_PDL(attn_decode_merge_kernel<D>, dim3(R, a.nq), splits >= MERGE_WIDE_FROM ? MERGE_THREADS : MERGE_THREADS / 2, 0,
                      stream, a);
    return SHARPI_OK;
}

// `splits` is the largest number of 256-key splits any served row needs; part_o / part_ml are
// scratch of [R, nq, splits, D] and [R, nq, splits, 2] floats.  `items` is an upper bound on the splits of all
// served rows together (0: R * splits); CTAs past the true total leave at once.
SHARPI_API int sharpi_attention_decode(const void* q, const void* kv, const int* block_table, const int* row_req,
                                       const int* positions, const int* rows, float* part_o, float* part_ml,
                                       void* out, int* status, int num_pages, int R, int nq, int nkv, int d,
                                       int max_blocks, int page_size, int mask_kind, int mask_span, int splits,
                                       int items, float scale, cudaStream_t stream) {
    if (R <= 0) return SHARPI_OK;
    if (nq <= 0 || nkv <= 0 || nq % nkv != 0 || page_size <= 0 || max_blocks <= 0 || splits <= 0 || R > 65535 ||
        nq > 65535)
        return SHARPI_BAD_ARGUMENT;
    if (mask_kind != SHARPI_MASK_FULL && mask_span <= 0) return SHARPI_BAD_ARGUMENT;
    if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(kv)) & 15) return SHARPI_UNALIGNED;
    DecodeArgs a;
    a.q = (const bf16*)q; a.kv = (const bf16*)kv; a.block_table = block_table; a.row_req = row_req;
    a.positions = positions; a.rows = rows; a.part_o = part_o; a.part_ml = part_ml; a.out = (bf16*)out;
    a.nq = nq; a.nkv = nkv; a.max_blocks = max_blocks; a.page_size = page_size; a.mask_kind = mask_kind;
    a.mask_span = mask_span; a.max_splits = splits; a.scale_log2 = scale * 1.4426950408889634f;
    a.num_rows = R;
    const long long all = (long long)R * splits;
    if (items <= 0 || items > all) items = (int)(all < 2147483647LL ? all : 2147483647LL);
    a.page_shift = -1;
    for (int sft = 0; sft < 31; ++sft)
        if ((1 << sft) == page_size) a.page_shift = sft;
    a.status = status;
    const long long pool_rows = (long long)num_pages * 2 * nkv * page_size;
    switch (d) {
        case 16: return launch_decode<16>(a, R, splits, items, pool_rows, stream);
        case 32: return launch_decode<32>(a, R, splits, items, pool_rows, stream);
        case 48: return launch_decode<48>(a, R, splits, items, pool_rows, stream);
        case 64: return launch_decode<64>(a, R, splits, items, pool_rows, stream);
        case 80: return launch_decode<80>(a, R, splits, items, pool_rows, stream);
        case 96: return launch_decode<96>(a, R, splits, items, pool_rows, stream);
        case 112: return launch_decode<112>(a, R, splits, items, pool_rows, stream);
        case 128: return launch_decode<128>(a, R, splits, items, pool_rows, stream);
        default: return SHARPI_BAD_ARGUMENT;   // other head sizes use the generic kernel
    }
}
