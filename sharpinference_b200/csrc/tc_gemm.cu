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
//   MODE_STORE   C[out_row, n] = (or +=) D            fp32, out_row = out_rows[sorted row] or the sorted row
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

using namespace sm100;

enum TcMode : int { MODE_STORE = 0, MODE_SWIGLU = 1 };

constexpr int TC_BM = 128;   // weight rows per tile (MMA M)
constexpr int TC_BK = 64;    // K elements per stage: 128 bytes, one swizzle row
constexpr int TC_THREADS = 192;

struct TcGemmParams {
    const int* group_offsets;   // [E + 1]
    const int* out_rows;        // MODE_STORE: nullable
    const float* row_scale;     // MODE_SWIGLU: nullable
    const int* scale_rows;      // MODE_SWIGLU: nullable
    void* out;                  // MODE_STORE: float [*, N]; MODE_SWIGLU: bf16 [rows, I]
    int* status;                // device word: 0 ok, else the code of the wait that gave up
    int rows, N, K, E;          // N: weight rows per expert (MODE_SWIGLU: 2 I)
    int accumulate;
    // K split over gridDim.z CTAs (few rows and few experts: not enough tiles to fill the GPU otherwise).
    // Each CTA then leaves its raw fp32 accumulators in partial[z][sorted row][N] and a second kernel adds
    // the parts in a fixed order and applies the epilogue.
    float* partial;
    int k_split;
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
    static constexpr int TMEM_COLS_NEEDED = W_TILES * NT;
    static constexpr int TMEM_COLS = TMEM_COLS_NEEDED <= 32 ? 32 : TMEM_COLS_NEEDED <= 64 ? 64 : TMEM_COLS_NEEDED <= 128 ? 128 : TMEM_COLS_NEEDED <= 256 ? 256 : 512;
};

template <int MODE, int NT, int WT>
__global__ void __launch_bounds__(TC_THREADS, 1)
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

    // ---- which tile is this CTA's ----------------------------------------------------------
    // Warp 0 looks the tile up: lane l reads the bounds of group e0 + l, the warp scans the tile counts, and
    // the group whose range of tiles holds blockIdx.y is the one (all loads at once, not a walk from group 0).
    if (warp == 0) {
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
            for (int s = 0; s < Cfg::STAGES; ++s) {
                mbar_init(&full_bar[s], 1);
                mbar_init(&empty_bar[s], 1);
            }
            mbar_init(accum_bar, 1);
            fence_barrier_init();
        }
    }
    __syncthreads();
    const int expert = tile_info[0];
    if (expert < 0) return;                       // uniform: nothing allocated yet
    const int row0 = tile_info[1], row_end = tile_info[2];
    // first weight row: MODE_SWIGLU: index into [0, I), the second tile is the matching up rows;
    // MODE_STORE: the second tile, if there is one, is the next 128 rows
    const int n0 = blockIdx.x * TC_BM * (MODE == MODE_SWIGLU ? 1 : WT);
    const int I = p.N / 2;                        // MODE_SWIGLU only
    const int n1 = (MODE == MODE_SWIGLU) ? I + n0 : n0 + TC_BM;
    const int k_blocks_all = (p.K + TC_BK - 1) / TC_BK;
    const int kb_per = (k_blocks_all + p.k_split - 1) / p.k_split;
    const int kb_begin = blockIdx.z * kb_per;
    const int k_blocks = max(0, min(k_blocks_all, kb_begin + kb_per) - kb_begin);   // this CTA's share

    if (warp == 5) {
        tmem_alloc(tmem_slot, Cfg::TMEM_COLS);
        tmem_relinquish();
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 4) {
        // ---- TMA producer ------------------------------------------------------------------
        if (lane == 0) {
            prefetch_tensormap(&map_w);
            prefetch_tensormap(&map_a);
            int issued = 0;
            bool ok = true;
            for (int kb = 0; kb < k_blocks && ok; ++kb) {
                const int s = kb % Cfg::STAGES;
                if (kb >= Cfg::STAGES) ok = mbar_wait(&empty_bar[s], ((kb / Cfg::STAGES) - 1) & 1);
                if (!ok) { atomicExch(p.status, 1); break; }
                uint8_t* stage = smem + s * Cfg::STAGE_BYTES;
                mbar_arrive_expect_tx(&full_bar[s], Cfg::STAGE_BYTES);
                const int kx = (kb_begin + kb) * TC_BK;
                tma_load_3d(stage, &map_w, &full_bar[s], kx, n0, expert);
                if (WT == 2) tma_load_3d(stage + Cfg::W_BYTES, &map_w, &full_bar[s], kx, n1, expert);
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
                ok = mbar_wait(&full_bar[s], (kb / Cfg::STAGES) & 1);
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
        const bool ok = mbar_wait(accum_bar, 0);
        if (!ok) {
            if (lane == 0) atomicExch(p.status, 3);
        } else {
            tcgen05_fence_after();
            const int n = n0 + warp * 32 + lane;
            const uint32_t lane_addr = tmem_base + ((uint32_t)(warp * 32) << 16);
            const int valid = min(NT, row_end - row0);
#pragma unroll 1
            for (int c0 = 0; c0 < NT; c0 += 16) {
                if (c0 >= valid) break;               // uniform over the warp
                float g[16];
                tmem_ld_16(lane_addr + c0, g);
                if (p.k_split > 1) {
                    float* part = p.partial + (size_t)blockIdx.z * p.rows * p.N;
                    float u[16];
                    if (WT == 2) tmem_ld_16(lane_addr + NT + c0, u);
                    const int nb = n1 - n0 + n;            // the row of the second tile
                    const bool n_ok = MODE == MODE_SWIGLU ? n < I : n < p.N;
                    const bool nb_ok = WT == 2 && (MODE == MODE_SWIGLU ? n < I : nb < p.N);
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const int r = row0 + c0 + j;
                        if (c0 + j < valid) {
                            if (n_ok) part[(size_t)r * p.N + n] = (k_blocks > 0) ? g[j] : 0.0f;
                            if (nb_ok) part[(size_t)r * p.N + nb] = (k_blocks > 0) ? u[j] : 0.0f;
                        }
                    }
                } else if (MODE == MODE_SWIGLU) {
                    float u[16];
                    tmem_ld_16(lane_addr + NT + c0, u);
                    if (n < I) {
                        bf16* act = reinterpret_cast<bf16*>(p.out);
                        float sc[16];                    // all the row scales first: the loads do not wait for stores
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            const int r = row0 + c0 + j;
                            sc[j] = (p.row_scale && c0 + j < valid) ? __ldg(p.row_scale + (p.scale_rows ? __ldg(p.scale_rows + r) : r))
                                                                     : 1.0f;
                        }
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            const int r = row0 + c0 + j;
                            if (c0 + j < valid) {
                                const float gv = g[j] * sc[j], uv = u[j] * sc[j];
                                act[(size_t)r * I + n] = __float2bfloat16_rn(gv / (1.0f + expf(-gv)) * uv);
                            }
                        }
                    }
                } else {
                    float* C = reinterpret_cast<float*>(p.out);
                    float u[16];
                    if (WT == 2) tmem_ld_16(lane_addr + NT + c0, u);
                    const bool n_ok = n < p.N, nb_ok = WT == 2 && n + TC_BM < p.N;
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const int r = row0 + c0 + j;
                        if (c0 + j < valid) {
                            // Adding in: every output element gets exactly one addend from this launch (a row
                            // belongs to one group), so a reduction that returns nothing gives the same sum
                            // as load, add, store, without a round trip to memory per element.
                            float* dst = C + (size_t)(p.out_rows ? p.out_rows[r] : r) * p.N + n;
                            if (p.accumulate) {
                                if (n_ok) atomicAdd(dst, g[j]);
                                if (nb_ok) atomicAdd(dst + TC_BM, u[j]);
                            } else {
                                if (n_ok) *dst = g[j];
                                if (nb_ok) dst[TC_BM] = u[j];
                            }
                        }
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
    tc_grouped_gemm_kernel<MODE, NT, WT><<<grid, TC_THREADS, Cfg::SMEM_BYTES, stream>>>(mw, ma, p);
    SHARPI_CHECK_LAUNCH();
    return SHARPI_OK;
}

// Second half of a K-split product: add the parts in the order z = 0, 1, ... and apply the epilogue.
template <int MODE>
__global__ void tc_split_reduce_kernel(const TcGemmParams p) {
    const int r = blockIdx.x;
    const int n = blockIdx.y * blockDim.x + threadIdx.x;
    const int n_out = (MODE == MODE_SWIGLU) ? p.N / 2 : p.N;
    if (n >= n_out) return;
    const size_t plane = (size_t)p.rows * p.N;
    const float* part = p.partial + (size_t)r * p.N;
    float g = 0.0f, u = 0.0f;
    for (int z = 0; z < p.k_split; ++z) {
        g += part[z * plane + n];
        if (MODE == MODE_SWIGLU) u += part[z * plane + n_out + n];
    }
    if (MODE == MODE_SWIGLU) {
        const float s = p.row_scale ? p.row_scale[p.scale_rows ? p.scale_rows[r] : r] : 1.0f;
        const float gv = g * s, uv = u * s;
        reinterpret_cast<bf16*>(p.out)[(size_t)r * n_out + n] = __float2bfloat16_rn(gv / (1.0f + expf(-gv)) * uv);
    } else {
        float* dst = reinterpret_cast<float*>(p.out) + (size_t)(p.out_rows ? p.out_rows[r] : r) * p.N + n;
        *dst = p.accumulate ? *dst + g : g;
    }
}

// A [rows, K] bf16 sorted by expert; W [E, N, K] bf16; see the file header for the two modes.
// `row_tile` (16, 32, 64, 128 or 256) is the number of activation rows one CTA takes.
// `k_split` > 1 (with `partial`, k_split * rows * N floats of scratch) cuts K over that many CTAs per tile.
SHARPI_API int sharpi_tc_grouped_gemm(const void* A, const void* W, const int* group_offsets, void* out,
                                      const int* out_rows, const float* row_scale, const int* scale_rows,
                                      int* status, float* partial, int rows, int N, int K, int E, int mode,
                                      int row_tile, int accumulate, int k_split, cudaStream_t stream) {
    if (rows <= 0 || N <= 0) return SHARPI_OK;
    if (K <= 0 || E <= 0 || K % 8 != 0) return SHARPI_BAD_ARGUMENT;          // TMA: rows 16-byte aligned
    if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(W)) & 15) return SHARPI_UNALIGNED;
    if (mode == MODE_SWIGLU && (N % 2 != 0)) return SHARPI_BAD_ARGUMENT;
    if (!status || !group_offsets) return SHARPI_BAD_ARGUMENT;
    CUtensorMap mw, ma;
    if (!tmap::make_bf16_map(&mw, W, (uint64_t)K, (uint64_t)N, (uint64_t)E, TC_BK, TC_BM)) return SHARPI_LAUNCH_FAILED;
    if (!tmap::make_bf16_map(&ma, A, (uint64_t)K, (uint64_t)rows, 0, TC_BK, (uint32_t)row_tile)) return SHARPI_LAUNCH_FAILED;
    TcGemmParams p;
    p.group_offsets = group_offsets; p.out_rows = out_rows; p.row_scale = row_scale; p.scale_rows = scale_rows;
    p.out = out; p.status = status; p.rows = rows; p.N = N; p.K = K; p.E = E; p.accumulate = accumulate;
    if (k_split < 1 || k_split > 16 || (k_split > 1 && !partial)) return SHARPI_BAD_ARGUMENT;
    p.partial = partial; p.k_split = k_split;
    const int n_out = (mode == MODE_SWIGLU) ? N / 2 : N;
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
    if (rc != SHARPI_OK || k_split == 1) return rc;
    dim3 rgrid(rows, (n_out + 255) / 256);
    if (mode == MODE_SWIGLU)
        tc_split_reduce_kernel<MODE_SWIGLU><<<rgrid, 256, 0, stream>>>(p);
    else
        tc_split_reduce_kernel<MODE_STORE><<<rgrid, 256, 0, stream>>>(p);
    SHARPI_CHECK_LAUNCH();
    return SHARPI_OK;
}

// out[r, :] = in[rows[r], :] for bf16 rows of width K (a multiple of 8): the activations sorted by
// expert, so that TMA can fetch an expert's rows as one tile.
__global__ void gather_rows_bf16_kernel(const uint4* __restrict__ in, const int* __restrict__ rows,
                                        uint4* __restrict__ out, int vec_per_row) {
    const int r = blockIdx.x;
    const uint4* src = in + (size_t)rows[r] * vec_per_row;
    uint4* dst = out + (size_t)r * vec_per_row;
    for (int i = threadIdx.x; i < vec_per_row; i += blockDim.x) dst[i] = src[i];
}

SHARPI_API int sharpi_gather_rows_bf16(const void* in, const int* rows, void* out, int R, int K, cudaStream_t stream) {
    if (R <= 0) return SHARPI_OK;
    if (K <= 0 || K % 8 != 0) return SHARPI_BAD_ARGUMENT;
    if ((reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(out)) & 15) return SHARPI_UNALIGNED;
    gather_rows_bf16_kernel<<<R, 128, 0, stream>>>((const uint4*)in, rows, (uint4*)out, K / 8);
    SHARPI_CHECK_LAUNCH();
    return SHARPI_OK;
}
