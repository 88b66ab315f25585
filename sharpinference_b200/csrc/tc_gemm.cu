// Grouped (per-expert) bf16 matrix products on the 5th-generation tensor cores: tcgen05.mma with
// the accumulator in tensor memory, operands staged in shared memory by TMA, one elected thread
// issuing the MMAs.  The reference runs each routed expert as per-token matvecs after choosing
// the expert on the host (src/SharpInference.Engine/CudaForwardPass.cs:5554-5578); here all of a
// step's rows, sorted by expert, go through one launch.
//
// Shape of the problem: rows sorted by expert (`group_offsets[e]` .. `group_offsets[e+1]`),
// activations A [rows, K] bf16, weights W [E, N, K] bf16, both K-major.  A routed expert sees few
// rows (1 .. a few hundred) and the work is streaming W once, so the MMA is laid out "swapped":
// the 128-row M side of the instruction holds 128 weight rows, the N side holds a tile of
// NT rows of activations (16 .. 256), and D[weight row, activation row] lives in tensor memory with
// the weight rows on the 128 lanes.  One CTA computes one (expert, 128 weight rows, NT activation
// rows) tile over all of K in steps of 64 elements.
//
// Two epilogues:
//   MODE_STORE   C[out_row, n] = (or +=) s D          fp32, out_row = out_rows[sorted row] or the sorted row,
//                s = row_scale[scale_rows[sorted row]] or 1 (a router that weights its experts' outputs)
//   MODE_SWIGLU  W holds gate rows [0, I) and up rows [I, 2I); the CTA accumulates the gate tile
//                and the matching up tile side by side and writes
//                act[sorted row, i] = silu(s g) * (s u) as bf16, s = row_scale[scale_rows[sorted row]]
//                (the router weight scales gate and up before the nonlinearity,
//                src/SharpInference.Engine/ForwardPass.cs:2082-2088).
//
// Warps: 0-3 read the accumulator (warp w owns TMEM lanes 32w .. 32w+31) and write the output;
// warp 4 issues the TMA loads; warp 5 allocates tensor memory and issues the MMAs.  Every
// mbarrier wait is bounded; on a timeout the kernel sets *status and winds down.
//
// Each output element is one fp32 accumulation over K in a fixed order inside the tensor core,
// independent of which tile or batch the row fell into.
#include "common.cuh"
#include "sm100.cuh"
#include "tensor_map.cuh"

#include <type_traits>

using namespace sm100;

enum TcMode : int { MODE_STORE = 0, MODE_SWIGLU = 1 };

constexpr int TC_BM = 128;   // weight rows per tile (MMA M)
constexpr int TC_BK = 64;    // K elements per stage: 128 bytes, one swizzle row
constexpr int TC_THREADS = 192;

struct TcGemmParams {
    const int* group_offsets;   // [E + 1]
    const int* out_rows;        // MODE_STORE: nullable
    const float* row_scale;     // nullable
    const int* scale_rows;      // nullable
    void* out;                  // MODE_STORE: float [*, N]; MODE_SWIGLU: bf16 [rows, I]
    int* status;                // device word: 0 ok, else the code of the wait that gave up
    int rows, N, K, E;          // N: weight rows per expert (MODE_SWIGLU: 2 I)
    int accumulate;
    // K split over gridDim.z CTAs (few rows and few experts: not enough tiles to fill the GPU otherwise).
    // Each CTA then leaves its raw fp32 accumulators in partial[z][sorted row][N]; the one that finishes last
    // adds the parts in the order of z and applies the epilogue.
    float* partial;
    int k_split;
    int* tickets;               // K split: one counter per tile, zero before the launch and again after it
    // Every wait of the tiled kernel polls at most this often before it gives up.  `drop_loads_from` >= 0 makes
    // the producer stop at that K block, so that the waits behind it run out: how a test sees a kernel give
    // up, record its code and return (see sharpi_tc_set_wait_test); -1 in every other launch.
    uint32_t wait_limit;
    int drop_loads_from;
};

// WT: weight tiles of 128 rows that share one activation tile.  MODE_SWIGLU always has two (gate and up);
// MODE_STORE takes two adjacent ones for large activation tiles, where the activations would otherwise be
// half of what the CTA holds in flight and the weights, which come from DRAM, the other half only.
template <int MODE, int NT, int WT>
struct TcConfig {
    static_assert(WT == 1 || WT == 2, "one or two weight tiles");
    static_assert(MODE != MODE_SWIGLU || WT == 2, "gate and up are two tiles");
    static constexpr int W_TILES = WT;
    static constexpr int W_BYTES = TC_BM * TC_BK * 2;
    static constexpr int A_BYTES = NT * TC_BK * 2;
    static constexpr int STAGE_BYTES = W_TILES * W_BYTES + A_BYTES;
    // stages: what fits 108 KB (so that two CTAs share an SM) for small tiles, 200 KB otherwise
    // (two CTAs with two 48 KB stages each measured faster than one CTA with four)
    static constexpr int BUDGET = (STAGE_BYTES <= 48 * 1024) ? 108 * 1024 : 200 * 1024;
    static constexpr int STAGES = (BUDGET / STAGE_BYTES) > 8 ? 8 : (BUDGET / STAGE_BYTES);
    static_assert(STAGES >= 2, "a tile configuration must leave room for two stages");
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*alignment*/ + 256 /*barriers*/;
    // registers are capped so that the two CTAs that fit an SM by shared memory also fit by registers
    static constexpr int MIN_CTAS = (2 * SMEM_BYTES <= 224 * 1024) ? 2 : 1;
    static constexpr int TMEM_COLS_NEEDED = W_TILES * NT;
    static constexpr int TMEM_COLS = TMEM_COLS_NEEDED <= 32 ? 32 : TMEM_COLS_NEEDED <= 64 ? 64 : TMEM_COLS_NEEDED <= 128 ? 128 : TMEM_COLS_NEEDED <= 256 ? 256 : 512;
};

// silu(g) * u with the exponential and the reciprocal as single instructions (relative error about 2^-21;
// the result is rounded to bfloat16).  Every epilogue of this file uses this one form.
__device__ __forceinline__ float silu_mul(float g, float u) {
    return g * rcp_approx(1.0f + ex2_approx(-1.4426950408889634f * g)) * u;
}

// The epilogue of 16 accumulator columns (sorted rows r_first .. r_first + 15, of which `count` exist) of one
// thread's weight row(s): g from the first weight tile (row n), u from the second (MODE_SWIGLU: the matching
// up row; MODE_STORE: row n + 128, if the CTA has a second tile).
template <int MODE>
__device__ __forceinline__ void tc_epilogue_chunk(const TcGemmParams& p, const float* g, const float* u, bool two_tiles,
                                                  int n, int r_first, int count) {
    // lane j of the warp fetches the scale of column j (all threads of a warp share the 16 columns)
    const int lane = threadIdx.x & 31;
    float mine = 1.0f;
    if (p.row_scale && lane < count) {
        const int r = r_first + lane;
        mine = p.row_scale[p.scale_rows ? p.scale_rows[r] : r];
    }
    float sc[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) sc[j] = __shfl_sync(0xffffffffu, mine, j);
    if (MODE == MODE_SWIGLU) {
        const int I = p.N / 2;
        if (n < I) {
            bf16* act = reinterpret_cast<bf16*>(p.out);
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                if (j < count) {
                    const float gv = g[j] * sc[j], uv = u[j] * sc[j];
                    act[(size_t)(r_first + j) * I + n] = __float2bfloat16_rn(silu_mul(gv, uv));
                }
            }
        }
    } else {
        float* C = reinterpret_cast<float*>(p.out);
        const bool n_ok = n < p.N, nb_ok = two_tiles && n + TC_BM < p.N;
        const bool scaled = p.row_scale != nullptr;      // a router that weights the experts' outputs
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            if (j < count) {
                // Adding in: every output element gets exactly one addend from this launch (a row belongs to
                // one group), so a reduction that returns nothing gives the same sum as load, add, store,
                // without a round trip to memory per element.
                const int r = r_first + j;
                float* dst = C + (size_t)(p.out_rows ? p.out_rows[r] : r) * p.N + n;
                const float gv = scaled ? g[j] * sc[j] : g[j], uv = scaled ? u[j] * sc[j] : u[j];
                if (p.accumulate) {
                    if (n_ok) atomicAdd(dst, gv);
                    if (nb_ok) atomicAdd(dst + TC_BM, uv);
                } else {
                    if (n_ok) *dst = gv;
                    if (nb_ok) dst[TC_BM] = uv;
                }
            }
        }
    }
}

template <int MODE, int NT, int WT>
__global__ void __launch_bounds__(TC_THREADS, TcConfig<MODE, NT, WT>::MIN_CTAS)
tc_grouped_gemm_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_a,
                       const TcGemmParams p) {
    using Cfg = TcConfig<MODE, NT, WT>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + Cfg::STAGES * Cfg::STAGE_BYTES);
    uint64_t* empty_bar = full_bar + Cfg::STAGES;
    uint64_t* accum_bar = empty_bar + Cfg::STAGES;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(accum_bar + 1);
    int* tile_info = reinterpret_cast<int*>(tmem_slot + 1);   // [0] expert, [1] first sorted row, [2] end row

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    // ---- set-up that touches nothing an earlier kernel writes: it may overlap that kernel's tail ----------
    const int n0 = blockIdx.x * TC_BM * (MODE == MODE_SWIGLU ? 1 : WT);    // first weight row (MODE_SWIGLU: in [0, I))
    const int I = p.N / 2;                                                 // MODE_SWIGLU only
    // the second tile: MODE_SWIGLU: the matching up rows; MODE_STORE: the next 128 rows, if the CTA has two
    const int n1 = (MODE == MODE_SWIGLU) ? I + n0 : n0 + TC_BM;
    const int k_blocks_all = (p.K + TC_BK - 1) / TC_BK;
    const int kb_per = (k_blocks_all + p.k_split - 1) / p.k_split;
    const int kb_begin = blockIdx.z * kb_per;
    const int k_blocks = max(0, min(k_blocks_all, kb_begin + kb_per) - kb_begin);   // this CTA's share
    // One group (a dense product): the tile follows from the block index alone, and the weights, which no
    // kernel writes, can be on their way into the first stages before the kernel ahead has finished.
    const bool dense = p.E == 1;
    const bool dense_tile = dense && (int)blockIdx.y * NT < p.rows;
    const int early = dense_tile ? min(k_blocks, Cfg::STAGES) : 0;
    if (threadIdx.x == 0) {
        for (int s = 0; s < Cfg::STAGES; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        mbar_init(accum_bar, 1);
        fence_barrier_init();
        if (dense) {
            tile_info[0] = dense_tile ? 0 : -1;
            tile_info[1] = blockIdx.y * NT;
            tile_info[2] = p.rows;
        }
    }
    if (warp == 5) {
        tmem_alloc(tmem_slot, Cfg::TMEM_COLS);
        tmem_relinquish();
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    if (warp == 4 && lane == 0) {
        prefetch_tensormap(&map_w);
        prefetch_tensormap(&map_a);
        for (int kb = 0; kb < early; ++kb) {
            uint8_t* stage = smem + kb * Cfg::STAGE_BYTES;
            mbar_arrive_expect_tx(&full_bar[kb], Cfg::STAGE_BYTES);       // the activations' bytes follow below
            const int kx = (kb_begin + kb) * TC_BK;
            tma_load_3d(stage, &map_w, &full_bar[kb], kx, n0, 0);
            if (WT == 2) tma_load_3d(stage + Cfg::W_BYTES, &map_w, &full_bar[kb], kx, n1, 0);
        }
    }
    pdl_wait();

    // ---- which tile is this CTA's ----------------------------------------------------------
    // Several groups: warp 0 looks the tile up: lane l reads the bounds of group e0 + l, the warp scans the tile
    // counts, and the group whose range of tiles holds blockIdx.y is the one (all loads at once, not a walk
    // from group 0).
    if (!dense && warp == 0) {
        const int tile = blockIdx.y;
        int found = -1, f_start = 0, f_end = 0, f_tile = 0, base = 0;
        for (int e0 = 0; e0 < p.E && found < 0; e0 += 32) {
            const int e = e0 + lane;
            int start = 0, end = 0;
            if (e < p.E) {
                start = p.group_offsets[e];
                end = p.group_offsets[e + 1];
            }
            const int tiles = (end - start + NT - 1) / NT;
            int incl = tiles;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int v = __shfl_up_sync(0xffffffffu, incl, o);
                if (lane >= o) incl += v;
            }
            const int first = base + incl - tiles;
            const unsigned hit = __ballot_sync(0xffffffffu, e < p.E && tile >= first && tile < first + tiles);
            if (hit) {
                const int src = __ffs(hit) - 1;
                found = e0 + src;
                f_start = __shfl_sync(0xffffffffu, start, src);
                f_end = __shfl_sync(0xffffffffu, end, src);
                f_tile = tile - __shfl_sync(0xffffffffu, first, src);
            }
            base += __shfl_sync(0xffffffffu, incl, 31);
        }
        if (lane == 0) {
            tile_info[0] = found;
            tile_info[1] = f_start + f_tile * NT;
            tile_info[2] = f_end;
        }
    }
    if (!dense) __syncthreads();
    const int expert = tile_info[0];
    const bool has_tile = expert >= 0;            // uniform over the CTA; without a tile only the exit is left
    const int row0 = tile_info[1], row_end = tile_info[2];

    if (!has_tile) {
        // nothing to do but to leave together
    } else if (warp == 4) {
        // ---- TMA producer ------------------------------------------------------------------
        if (lane == 0) {
            int issued = 0;
            bool ok = true;
            for (int kb = 0; kb < k_blocks && ok; ++kb) {
                if (p.drop_loads_from >= 0 && kb >= p.drop_loads_from) break;     // test only: see TcGemmParams
                const int s = kb % Cfg::STAGES;
                if (kb >= Cfg::STAGES) ok = mbar_wait(&empty_bar[s], ((kb / Cfg::STAGES) - 1) & 1, p.wait_limit);
                if (!ok) { atomicExch(p.status, 1); break; }
                uint8_t* stage = smem + s * Cfg::STAGE_BYTES;
                const int kx = (kb_begin + kb) * TC_BK;
                if (kb >= early) {                    // else the weights of this stage are on their way already
                    mbar_arrive_expect_tx(&full_bar[s], Cfg::STAGE_BYTES);
                    tma_load_3d(stage, &map_w, &full_bar[s], kx, n0, expert);
                    if (WT == 2) tma_load_3d(stage + Cfg::W_BYTES, &map_w, &full_bar[s], kx, n1, expert);
                }
                tma_load_2d(stage + Cfg::W_TILES * Cfg::W_BYTES, &map_a, &full_bar[s], kx, row0);
                issued = kb + 1;
            }
            if (!ok) {
                // let the copies that were started land before the block goes away
                for (int kb = max(0, issued - Cfg::STAGES); kb < issued; ++kb)
                    mbar_wait(&full_bar[kb % Cfg::STAGES], (kb / Cfg::STAGES) & 1, 1u << 16);
            }
        }
    } else if (warp == 5) {
        // ---- MMA issuer --------------------------------------------------------------------
        if (lane == 0) {
            const uint32_t idesc = instr_desc_bf16(TC_BM, NT);
            bool ok = true;
            for (int kb = 0; kb < k_blocks; ++kb) {
                const int s = kb % Cfg::STAGES;
                ok = mbar_wait(&full_bar[s], (kb / Cfg::STAGES) & 1, p.wait_limit);
                if (!ok) { atomicExch(p.status, 2); break; }
                tcgen05_fence_after();
                const uint8_t* stage = smem + s * Cfg::STAGE_BYTES;
                const uint8_t* a_tile = stage + Cfg::W_TILES * Cfg::W_BYTES;
#pragma unroll
                for (int k = 0; k < TC_BK / 16; ++k) {
                    const uint32_t acc = (kb | k) != 0;
                    const uint64_t db = smem_desc_k_sw128(a_tile, k * 32);
                    mma_bf16_ss(tmem_base, smem_desc_k_sw128(stage, k * 32), db, idesc, acc);
                    if (WT == 2)
                        mma_bf16_ss(tmem_base + NT, smem_desc_k_sw128(stage + Cfg::W_BYTES, k * 32), db, idesc, acc);
                }
                mma_commit(&empty_bar[s]);      // the stage is free when these MMAs have read it
            }
            if (ok) mma_commit(accum_bar);       // the accumulator is complete
        }
    } else {
        // ---- epilogue: warps 0..3, thread = TMEM lane = weight row ---------------------------
        const bool ok = mbar_wait(accum_bar, 0, p.wait_limit);
        const int n = n0 + warp * 32 + lane;
        const int nb = n1 - n0 + n;                    // the row of the second tile
        const int valid = min(NT, row_end - row0);
        const size_t plane = (size_t)p.rows * p.N;
        const bool n_ok = MODE == MODE_SWIGLU ? n < I : n < p.N;
        const bool nb_ok = WT == 2 && (MODE == MODE_SWIGLU ? n < I : nb < p.N);
        if (!ok) {
            if (lane == 0) atomicExch(p.status, 3);
        } else {
            tcgen05_fence_after();
            const uint32_t lane_addr = tmem_base + ((uint32_t)(warp * 32) << 16);
#pragma unroll 1
            for (int c0 = 0; c0 < NT; c0 += 16) {
                if (c0 >= valid) break;               // uniform over the warp
                float g[16], u[16];
                tmem_ld_16(lane_addr + c0, g);
                if (WT == 2) tmem_ld_16(lane_addr + NT + c0, u);
                if (p.k_split > 1) {
                    float* part = p.partial + (size_t)blockIdx.z * plane;
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const int r = row0 + c0 + j;
                        if (c0 + j < valid) {
                            if (n_ok) part[(size_t)r * p.N + n] = (k_blocks > 0) ? g[j] : 0.0f;
                            if (nb_ok) part[(size_t)r * p.N + nb] = (k_blocks > 0) ? u[j] : 0.0f;
                        }
                    }
                } else {
                    tc_epilogue_chunk<MODE>(p, g, u, WT == 2, n, row0 + c0, min(16, valid - c0));
                }
            }
        }
        if (p.k_split > 1) {
            // The CTA that finishes last of the tile's K parts adds them, in the order of the parts, and applies
            // the epilogue.  All 128 threads meet at a barrier of their own that also tells whether all of them
            // have their part (a wait that gave up must not leave the others waiting here).
            __threadfence();
            if (named_barrier_all(1, 128, ok)) {
                if (threadIdx.x == 0) {
                    int* ticket = p.tickets + (size_t)blockIdx.y * gridDim.x + blockIdx.x;
                    const int last = atomicAdd(ticket, 1) == p.k_split - 1;
                    if (last) *ticket = 0;
                    tile_info[3] = last;
                }
                named_barrier_all(1, 128, true);
                if (tile_info[3]) {
                    __threadfence();
#pragma unroll 1
                    for (int c0 = 0; c0 < valid; c0 += 16) {
                        float g[16], u[16];
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            g[j] = 0.0f;
                            u[j] = 0.0f;
                        }
                        for (int z = 0; z < p.k_split; ++z) {
                            const float* part = p.partial + (size_t)z * plane;
#pragma unroll
                            for (int j = 0; j < 16; ++j) {
                                const int r = row0 + c0 + j;
                                if (c0 + j < valid) {
                                    if (n_ok) g[j] += __ldcg(part + (size_t)r * p.N + n);
                                    if (nb_ok) u[j] += __ldcg(part + (size_t)r * p.N + nb);
                                }
                            }
                        }
                        tc_epilogue_chunk<MODE>(p, g, u, WT == 2, n, row0 + c0, min(16, valid - c0));
                    }
                }
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

// ---------------------------------------------------------------------------------------
// Persistent variant for steps with many rows (prompts).
//
// One CTA per SM walks a list of work items: (group, chunk of up to 256 of its rows, two weight tiles of 128
// rows).  An item streams its two weight tiles over all of K once and multiplies them with one or two
// activation tiles of 128 rows, so a group of up to 256 rows reads its weights once (the kernel above gives
// every 128 rows a CTA of their own, which streams the weights again).  The three roles run ahead of one
// another across items: the producer fills a ring of four weight stages and six activation slots, the MMA
// warp accumulates into tensor memory, the epilogue warps drain it.  Tensor memory (512 columns) holds two
// items of up to 128 rows at once, one being multiplied while the other is drained, or one of up to 256.
// The N extent of each MMA is the number of rows rounded up to 16, so short groups cost what they hold.
// Items go to CTAs round-robin; items next to each other share a group, so its activations stay in L2.
// Each output element is still one accumulation over K in ascending order inside the tensor core.
// ---------------------------------------------------------------------------------------
// Two shapes of the rings, both 224 KB: four weight stages and six activation slots when the kernel has every SM
// (a CTA then needs 128 KB of weights in flight), five and four when it is given a part of the SMs and the rest
// run another kernel beside it (fewer CTAs must keep the same memory stream going: 160 KB in flight each).
constexpr int PS_W_BYTES = 2 * TC_BM * TC_BK * 2;   // two weight tiles: 32 KB
constexpr int PS_A_BYTES = 128 * TC_BK * 2;         // 128 activation rows: 16 KB
constexpr int PS_CHUNK = 256;                       // rows per item
constexpr int PS_MAX_E = 256;                       // groups whose bounds fit the shared-memory table
constexpr int PS_TABLE_BYTES = 2 * (PS_MAX_E + 1) * 4;
constexpr int PS_SMEM = 224 * 1024 + 256 + PS_TABLE_BYTES;
static_assert(PS_SMEM <= 227 * 1024, "the persistent kernel's rings must fit one CTA");

struct PsItem {
    int expert, row0, nrows, n_tile;
};

// Item w of the list: groups in order, their chunks in order, the weight tiles of a chunk next to each other.
// `e` is a cursor that only moves forward (a CTA's items ascend).
__device__ __forceinline__ PsItem ps_decode(int w, int& e, const int* first_s, const int* off_s, int n_tiles) {
    while (w >= first_s[e + 1]) ++e;
    const int local = w - first_s[e];
    PsItem it;
    it.expert = e;
    it.n_tile = local % n_tiles;
    it.row0 = off_s[e] + (local / n_tiles) * PS_CHUNK;
    it.nrows = min(PS_CHUNK, off_s[e + 1] - it.row0);
    return it;
}

constexpr int PS_EPI_WARPS = 8;                     // two per quarter of the tensor-memory lanes
constexpr int PS_THREADS = (PS_EPI_WARPS + 2) * 32;  // then the producer warp and the MMA warp

template <int MODE, int PS_W_STAGES, int PS_A_SLOTS>
__global__ void __launch_bounds__(PS_THREADS, 1)
tc_grouped_gemm_persistent_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_a,
                                  const TcGemmParams p) {
    static_assert(PS_W_STAGES * PS_W_BYTES + PS_A_SLOTS * PS_A_BYTES == 224 * 1024, "the rings take 224 KB");
    static_assert(PS_W_STAGES + PS_A_SLOTS + PS_W_STAGES + PS_A_SLOTS + 4 <= 31, "barriers and the slot fit 256 bytes");
    extern __shared__ __align__(1024) uint8_t ps_smem[];
    if (smem_u32(ps_smem) & 1023u) {             // the swizzled tiles need it; nothing has been set up yet
        if (threadIdx.x == 0) atomicExch(p.status, 6);
        return;
    }
    uint8_t* w_ring = ps_smem;
    uint8_t* a_ring = w_ring + PS_W_STAGES * PS_W_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(a_ring + PS_A_SLOTS * PS_A_BYTES);
    uint64_t* full_w = bars;                      // [4]
    uint64_t* empty_w = full_w + PS_W_STAGES;     // [4]
    uint64_t* full_a = empty_w + PS_W_STAGES;     // [6]
    uint64_t* empty_a = full_a + PS_A_SLOTS;      // [6]
    uint64_t* full_t = empty_a + PS_A_SLOTS;      // [2] accumulators of a half of tensor memory complete
    uint64_t* empty_t = full_t + 2;               // [2] ... drained (128 arrivals)
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(empty_t + 2);
    int* first_s = reinterpret_cast<int*>(reinterpret_cast<uint8_t*>(bars) + 256);   // [E + 1] first item of a group
    int* off_s = first_s + PS_MAX_E + 1;                                              // [E + 1] first row of a group

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int I = p.N / 2;
    const int n_tiles = (MODE == MODE_SWIGLU) ? (I + TC_BM - 1) / TC_BM : (p.N + 2 * TC_BM - 1) / (2 * TC_BM);
    const int k_blocks = (p.K + TC_BK - 1) / TC_BK;

    if (warp == 0) {
        int base = 0;
        for (int e0 = 0; e0 < p.E; e0 += 32) {
            const int e = e0 + lane;
            int start = 0, end = 0;
            if (e < p.E) {
                start = p.group_offsets[e];
                end = p.group_offsets[e + 1];
            }
            const int items = ((end - start + PS_CHUNK - 1) / PS_CHUNK) * n_tiles;
            int incl = items;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int v = __shfl_up_sync(0xffffffffu, incl, o);
                if (lane >= o) incl += v;
            }
            if (e < p.E) {
                first_s[e] = base + incl - items;
                off_s[e] = start;
            }
            base += __shfl_sync(0xffffffffu, incl, 31);
        }
        if (lane == 0) {
            first_s[p.E] = base;
            off_s[p.E] = p.group_offsets[p.E];
            for (int i = 0; i < PS_W_STAGES; ++i) { mbar_init(&full_w[i], 1); mbar_init(&empty_w[i], 1); }
            for (int i = 0; i < PS_A_SLOTS; ++i) { mbar_init(&full_a[i], 1); mbar_init(&empty_a[i], 1); }
            for (int i = 0; i < 2; ++i) { mbar_init(&full_t[i], 1); mbar_init(&empty_t[i], PS_EPI_WARPS * 32); }
            fence_barrier_init();
        }
    }
    if (warp == PS_EPI_WARPS + 1) {
        tmem_alloc(tmem_slot, 512);
        tmem_relinquish();
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const int total = first_s[p.E];

    if (warp == PS_EPI_WARPS) {
        // ---- TMA producer ------------------------------------------------------------------
        if (lane == 0) {
            prefetch_tensormap(&map_w);
            prefetch_tensormap(&map_a);
            uint32_t cw = 0, ca = 0;          // weight stages and activation slots filled so far
            int e = 0;
            bool ok = true;
            for (int w = blockIdx.x; w < total && ok; w += gridDim.x) {
                const PsItem it = ps_decode(w, e, first_s, off_s, n_tiles);
                const int n0 = it.n_tile * TC_BM * (MODE == MODE_SWIGLU ? 1 : 2);
                const int n1 = (MODE == MODE_SWIGLU) ? I + n0 : n0 + TC_BM;
                const int subs = (it.nrows + 127) >> 7;
                for (int kb = 0; kb < k_blocks && ok; ++kb) {
                    const int kx = kb * TC_BK;
                    const int ws = cw % PS_W_STAGES;
                    if (cw >= PS_W_STAGES) ok = mbar_wait(&empty_w[ws], ((cw / PS_W_STAGES) - 1) & 1);
                    if (!ok) { atomicExch(p.status, 1); break; }
                    uint8_t* wt = w_ring + ws * PS_W_BYTES;
                    mbar_arrive_expect_tx(&full_w[ws], PS_W_BYTES);
                    tma_load_3d(wt, &map_w, &full_w[ws], kx, n0, it.expert);
                    tma_load_3d(wt + PS_W_BYTES / 2, &map_w, &full_w[ws], kx, n1, it.expert);
                    ++cw;
                    for (int sub = 0; sub < subs; ++sub) {
                        const int as = ca % PS_A_SLOTS;
                        if (ca >= PS_A_SLOTS) ok = mbar_wait(&empty_a[as], ((ca / PS_A_SLOTS) - 1) & 1);
                        if (!ok) { atomicExch(p.status, 1); break; }
                        mbar_arrive_expect_tx(&full_a[as], PS_A_BYTES);
                        tma_load_2d(a_ring + as * PS_A_BYTES, &map_a, &full_a[as], kx, it.row0 + sub * 128);
                        ++ca;
                    }
                }
            }
            if (!ok) {
                // let the copies that were started land before the block goes away
                for (uint32_t c = cw > PS_W_STAGES ? cw - PS_W_STAGES : 0; c < cw; ++c)
                    mbar_wait(&full_w[c % PS_W_STAGES], (c / PS_W_STAGES) & 1, 1u << 16);
                for (uint32_t c = ca > PS_A_SLOTS ? ca - PS_A_SLOTS : 0; c < ca; ++c)
                    mbar_wait(&full_a[c % PS_A_SLOTS], (c / PS_A_SLOTS) & 1, 1u << 16);
            }
        }
    } else if (warp == PS_EPI_WARPS + 1) {
        // ---- MMA issuer --------------------------------------------------------------------
        // One thread issues every MMA of the CTA, so its instruction stream is kept short: ring positions and
        // parities advance by increments, descriptors are a base plus the position times the slot size.
        if (lane == 0) {
            uint32_t ws = 0, pw = 0, as = 0, pa = 0;       // weight stage / activation slot and their parities
            uint32_t use0 = 0, use1 = 0;
            int e = 0, next_half = 0;
            bool ok = true;
            const uint64_t wdesc = smem_desc_k_sw128(w_ring, 0), adesc = smem_desc_k_sw128(a_ring, 0);
            auto run_item = [&](auto subs_tag, const PsItem& it, uint32_t acc_base) {
                constexpr int SUBS = decltype(subs_tag)::value;
                const uint32_t idesc0 = instr_desc_bf16(TC_BM, (min(128, it.nrows) + 15) & ~15);
                const uint32_t idesc1 = SUBS == 2 ? instr_desc_bf16(TC_BM, (it.nrows - 128 + 15) & ~15) : 0u;
                for (int kb = 0; kb < k_blocks; ++kb) {
                    if (!mbar_wait(&full_w[ws], pw)) return false;
                    const uint32_t as1 = (as + 1 == PS_A_SLOTS) ? 0 : as + 1;
                    if (!mbar_wait(&full_a[as], pa)) return false;
                    if (SUBS == 2 && !mbar_wait(&full_a[as1], as1 == 0 ? pa ^ 1 : pa)) return false;
                    tcgen05_fence_after();
                    const uint64_t dw0 = wdesc + (uint64_t)(ws * (PS_W_BYTES >> 4));
                    const uint64_t dw1 = dw0 + (uint64_t)(PS_W_BYTES >> 5);
                    const uint64_t da0 = adesc + (uint64_t)(as * (PS_A_BYTES >> 4));
                    const uint64_t da1 = adesc + (uint64_t)(as1 * (PS_A_BYTES >> 4));
#pragma unroll
                    for (int k = 0; k < TC_BK / 16; ++k) {
                        const uint32_t acc = (kb | k) != 0;
                        // alternate the accumulators: back-to-back MMAs into one accumulator wait for each other
                        mma_bf16_ss(acc_base, dw0 + 2 * k, da0 + 2 * k, idesc0, acc);
                        mma_bf16_ss(acc_base + 128, dw1 + 2 * k, da0 + 2 * k, idesc0, acc);
                        if (SUBS == 2) {          // the second 128 rows accumulate in the other half
                            mma_bf16_ss(acc_base + 256, dw0 + 2 * k, da1 + 2 * k, idesc1, acc);
                            mma_bf16_ss(acc_base + 256 + 128, dw1 + 2 * k, da1 + 2 * k, idesc1, acc);
                        }
                    }
                    mma_commit(&empty_w[ws]);         // free when these MMAs have read them
                    mma_commit(&empty_a[as]);
                    if (SUBS == 2) mma_commit(&empty_a[as1]);
                    ws = (ws + 1 == PS_W_STAGES) ? 0 : ws + 1;
                    pw ^= (ws == 0);
                    as += SUBS;
                    if (as >= PS_A_SLOTS) { as -= PS_A_SLOTS; pa ^= 1; }
                }
                return true;
            };
            for (int w = blockIdx.x; w < total && ok; w += gridDim.x) {
                const PsItem it = ps_decode(w, e, first_s, off_s, n_tiles);
                const bool big = it.nrows > 128;
                // an item of up to 128 rows takes one half of tensor memory (the halves alternate), a larger one both
                const int h0 = big ? 0 : next_half;
                next_half = big ? 0 : next_half ^ 1;
                if ((big || h0 == 0) && use0 > 0) ok = mbar_wait(&empty_t[0], (use0 - 1) & 1);
                if (ok && (big || h0 == 1) && use1 > 0) ok = mbar_wait(&empty_t[1], (use1 - 1) & 1);
                if (!ok) { atomicExch(p.status, 7); break; }
                tcgen05_fence_after();
                const uint32_t acc_base = tmem_base + h0 * 256;
                ok = big ? run_item(std::integral_constant<int, 2>{}, it, acc_base)
                         : run_item(std::integral_constant<int, 1>{}, it, acc_base);
                if (!ok) { atomicExch(p.status, 2); break; }
                if (big || h0 == 0) { mma_commit(&full_t[0]); ++use0; }     // the item's accumulators are complete
                if (big || h0 == 1) { mma_commit(&full_t[1]); ++use1; }
            }
        }
    } else {
        // ---- epilogue: warps 0..7; warp w reads lanes 32 (w % 4) .. (thread = weight row) and every second
        // 16-column piece, starting at piece w / 4.  A half of tensor memory is handed back as soon as its 128
        // rows are out, so the next item can start while the second half of a large item is still drained.
        uint32_t uses[2] = {0, 0};
        int e = 0, next_half = 0;
        bool ok = true;
        const uint32_t lane_base = tmem_base + ((uint32_t)((warp & 3) * 32) << 16);
        for (int w = blockIdx.x; w < total && ok; w += gridDim.x) {
            const PsItem it = ps_decode(w, e, first_s, off_s, n_tiles);
            const int subs = (it.nrows + 127) >> 7;
            const int h0 = (subs == 2) ? 0 : next_half;
            next_half = (subs == 2) ? 0 : next_half ^ 1;
            const int n = it.n_tile * TC_BM * (MODE == MODE_SWIGLU ? 1 : 2) + (warp & 3) * 32 + lane;
            for (int sub = 0; sub < subs && ok; ++sub) {
                const int h = h0 + sub;
                ok = mbar_wait(&full_t[h], uses[h] & 1);
                if (!ok) {
                    if (lane == 0) atomicExch(p.status, 3);
                    break;
                }
                tcgen05_fence_after();
                const uint32_t acc = lane_base + h * 256;
                const int valid = min(128, it.nrows - sub * 128);
#pragma unroll 1
                for (int c0 = (warp >> 2) * 16; c0 < valid; c0 += 32) {
                    float g[16], u[16];
                    tmem_ld_16(acc + c0, g);
                    tmem_ld_16(acc + 128 + c0, u);
                    tc_epilogue_chunk<MODE>(p, g, u, true, n, it.row0 + sub * 128 + c0, min(16, valid - c0));
                }
                tcgen05_fence_before();
                mbar_arrive(&empty_t[h]);
                ++uses[h];
            }
        }
    }
    tcgen05_fence_before();
    __syncthreads();
    if (warp == PS_EPI_WARPS + 1) {
        tcgen05_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
}

// `max_ctas` > 0 gives the kernel that many SMs at most (and the deeper weight ring); 0: every SM.
template <int MODE, int WS, int AS>
static int launch_persistent(const CUtensorMap& mw, const CUtensorMap& ma, const TcGemmParams& p, long long max_items,
                             int max_ctas, cudaStream_t stream) {
    static bool configured = false;
    static int sms = 0;
    if (!configured) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess ||
            cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
            return SHARPI_LAUNCH_FAILED;
        if (cudaFuncSetAttribute(tc_grouped_gemm_persistent_kernel<MODE, WS, AS>,
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, PS_SMEM) != cudaSuccess)
            return SHARPI_LAUNCH_FAILED;
        configured = true;
    }
    long long grid = max_items < sms ? max_items : sms;
    if (max_ctas > 0 && grid > max_ctas) grid = max_ctas;
    tc_grouped_gemm_persistent_kernel<MODE, WS, AS><<<(int)grid, PS_THREADS, PS_SMEM, stream>>>(mw, ma, p);
    SHARPI_CHECK_LAUNCH();
    return SHARPI_OK;
}

// ---------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------
template <int MODE, int NT, int WT>
static int launch(const CUtensorMap& mw, const CUtensorMap& ma, const TcGemmParams& p, int n_tiles, int row_tiles,
                  cudaStream_t stream) {
    using Cfg = TcConfig<MODE, NT, WT>;
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(tc_grouped_gemm_kernel<MODE, NT, WT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 Cfg::SMEM_BYTES) != cudaSuccess)
            return SHARPI_LAUNCH_FAILED;
        configured = true;
    }
    dim3 grid(n_tiles, row_tiles, p.k_split);
    auto kern = tc_grouped_gemm_kernel<MODE, NT, WT>;
    SHARPI_LAUNCH_PDL(kern, grid, TC_THREADS, Cfg::SMEM_BYTES, stream, mw, ma, p);
    return SHARPI_OK;
}

// Test hook: the NEXT launch of sharpi_tc_grouped_gemm (tiled kernel) polls every wait at most `limit` times
// and its producer issues no loads from K block `drop_from` on.  The waits behind the missing loads run out,
// the kernel records the code of a wait that gave up in *status and returns with its tensor memory freed:
// the way a test observes that path without a fault.  The hook is consumed by that one launch.
static uint32_t g_test_wait_limit = 0;
static int g_test_drop_from = -1;

SHARPI_API void sharpi_tc_set_wait_test(unsigned limit, int drop_from) {
    g_test_wait_limit = limit;
    g_test_drop_from = drop_from;
}

// A [rows, K] bf16 sorted by expert; W [E, N, K] bf16; see the file header for the two modes.
// `row_tile` (16, 32, 64, 128 or 256) is the number of activation rows one CTA takes; 0 asks for the
// persistent kernel (up to 256 groups, no K split), which `max_ctas` > 0 keeps to that many SMs.
// `k_split` > 1 (with `partial`, k_split * rows * N floats of scratch, and `tickets`, one zero int per tile of the
// launch grid) cuts K over that many CTAs per tile.
SHARPI_API int sharpi_tc_grouped_gemm(const void* A, const void* W, const int* group_offsets, void* out,
                                      const int* out_rows, const float* row_scale, const int* scale_rows,
                                      int* status, float* partial, int* tickets, int rows, int N, int K, int E, int mode,
                                      int row_tile, int accumulate, int k_split, int max_ctas, cudaStream_t stream) {
    if (rows <= 0 || N <= 0) return SHARPI_OK;
    if (K <= 0 || E <= 0 || K % 8 != 0) return SHARPI_BAD_ARGUMENT;          // TMA: rows 16-byte aligned
    if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(W)) & 15) return SHARPI_UNALIGNED;
    if (mode == MODE_SWIGLU && (N % 2 != 0)) return SHARPI_BAD_ARGUMENT;
    if (!status || !group_offsets) return SHARPI_BAD_ARGUMENT;
    CUtensorMap mw, ma;
    if (!tmap::make_bf16_map(&mw, W, (uint64_t)K, (uint64_t)N, (uint64_t)E, TC_BK, TC_BM)) return SHARPI_LAUNCH_FAILED;
    if (!tmap::make_bf16_map(&ma, A, (uint64_t)K, (uint64_t)rows, 0, TC_BK, (uint32_t)(row_tile ? row_tile : 128)))
        return SHARPI_LAUNCH_FAILED;
    TcGemmParams p;
    p.group_offsets = group_offsets; p.out_rows = out_rows; p.row_scale = row_scale; p.scale_rows = scale_rows;
    p.out = out; p.status = status; p.rows = rows; p.N = N; p.K = K; p.E = E; p.accumulate = accumulate;
    if (k_split < 1 || k_split > 16 || (k_split > 1 && (!partial || !tickets))) return SHARPI_BAD_ARGUMENT;
    p.partial = partial; p.k_split = k_split; p.tickets = tickets;
    p.wait_limit = g_test_wait_limit ? g_test_wait_limit : WAIT_LIMIT;
    p.drop_loads_from = g_test_drop_from;
    g_test_wait_limit = 0;
    g_test_drop_from = -1;
    const int n_out = (mode == MODE_SWIGLU) ? N / 2 : N;
    if (row_tile == 0) {
        // the persistent kernel: 128-row activation boxes, two weight tiles per item
        if (k_split != 1 || E > PS_MAX_E || rows < 128) return SHARPI_BAD_ARGUMENT;
        const long long tiles = (mode == MODE_SWIGLU) ? (n_out + TC_BM - 1) / TC_BM : (N + 2 * TC_BM - 1) / (2 * TC_BM);
        const long long max_items = ((long long)rows / PS_CHUNK + (rows < E ? rows : E)) * tiles;
        if (max_ctas > 0)
            return mode == MODE_SWIGLU ? launch_persistent<MODE_SWIGLU, 5, 4>(mw, ma, p, max_items, max_ctas, stream)
                                       : launch_persistent<MODE_STORE, 5, 4>(mw, ma, p, max_items, max_ctas, stream);
        return mode == MODE_SWIGLU ? launch_persistent<MODE_SWIGLU, 4, 6>(mw, ma, p, max_items, 0, stream)
                                   : launch_persistent<MODE_STORE, 4, 6>(mw, ma, p, max_items, 0, stream);
    }
    // two weight tiles per activation tile pay from about 2048 rows on (measured at 16 experts: 281 vs 315 us
    // at 2048 rows, 658 vs 719 us at 8192; below that the larger number of CTAs of single tiles wins)
    const int store_wt = (mode == MODE_STORE && row_tile >= 128 && rows >= 2048) ? 2 : 1;
    const int n_tiles = (n_out + TC_BM * store_wt - 1) / (TC_BM * store_wt);
    // tiles = sum over experts of ceil(rows_e / row_tile) <= (experts with rows) + rows / row_tile, and at
    // most min(rows, E) experts have rows: no more CTAs than that are launched (empty ones cost a slot each)
    const long long row_tiles = rows / row_tile + (rows < E ? rows : E);
    if (row_tiles > 65535) return SHARPI_BAD_ARGUMENT;
    int rc = SHARPI_BAD_ARGUMENT;
#define TC_CASE(M, T, W) \
    if (mode == M && row_tile == T && (M == MODE_SWIGLU || store_wt == W)) \
        rc = launch<M, T, W>(mw, ma, p, n_tiles, (int)row_tiles, stream);
    TC_CASE(MODE_STORE, 16, 1) TC_CASE(MODE_STORE, 32, 1) TC_CASE(MODE_STORE, 64, 1) TC_CASE(MODE_STORE, 128, 1)
    TC_CASE(MODE_STORE, 128, 2) TC_CASE(MODE_STORE, 256, 1) TC_CASE(MODE_STORE, 256, 2)
    TC_CASE(MODE_SWIGLU, 16, 2) TC_CASE(MODE_SWIGLU, 32, 2) TC_CASE(MODE_SWIGLU, 64, 2) TC_CASE(MODE_SWIGLU, 128, 2)
    TC_CASE(MODE_SWIGLU, 256, 2)
#undef TC_CASE
    return rc;
}

// out[r, :] = in[rows[r], :] for bf16 rows of width K (a multiple of 8): the activations sorted by
// expert, so that TMA can fetch an expert's rows as one tile.
__global__ void gather_rows_bf16_kernel(const uint4* __restrict__ in, const int* __restrict__ rows,
                                        uint4* __restrict__ out, int vec_per_row) {
    pdl_wait();
    const int r = blockIdx.x;
    const uint4* src = in + (size_t)rows[r] * vec_per_row;
    uint4* dst = out + (size_t)r * vec_per_row;
    for (int i = threadIdx.x; i < vec_per_row; i += blockDim.x) dst[i] = src[i];
}

SHARPI_API int sharpi_gather_rows_bf16(const void* in, const int* rows, void* out, int R, int K, cudaStream_t stream) {
    if (R <= 0) return SHARPI_OK;
    if (K <= 0 || K % 8 != 0) return SHARPI_BAD_ARGUMENT;
    if ((reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(out)) & 15) return SHARPI_UNALIGNED;
    SHARPI_LAUNCH_PDL(gather_rows_bf16_kernel, R, 128, 0, stream, (const uint4*)in, rows, (uint4*)out, K / 8);
    return SHARPI_OK;
}
