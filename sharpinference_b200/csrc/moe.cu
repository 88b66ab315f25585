// Expert routing on the device: router logits, gate, top-1 choice, and the sort of the
// step's rows by expert.  Nothing comes back to the host; the reference downloads the
// router output and picks the expert on the CPU after a synchronize, once per layer and
// token (src/SharpInference.Engine/CudaForwardPass.cs:5532-5541).
//
// Formula (src/SharpInference.Engine/ForwardPass.cs:2027-2040, :2132-2163): r = h . Wr^T,
// p = sigmoid(r) elementwise, e* = the first index of the largest p (strict >), w = p[e*],
// no renormalisation for one expert per token.  The logits are fp32 dot products of the
// fp32 normalised activations with fp32 router weights, each summed in an order that the
// width alone fixes, so a token picks the same expert in every batch.
#include "common.cuh"

enum RouterGate : int {
    ROUTER_GATE_SIGMOID = 0,
};

constexpr int ROUTER_SEGMENTS = 8;

// The one summation order of a router logit, whatever kernel computes it: the width is cut into
// ROUTER_SEGMENTS contiguous segments (of a multiple of 4 elements); inside a segment a lane adds its own
// stride-32 pieces in ascending order (four-element pieces when `vec`), the warp adds the 32 lane sums in
// a fixed tree; the segment sums are added in ascending order.  So a token's logits are the same bits
// alone or in a large batch, and it picks the same expert in every way of cutting the work.
__host__ __device__ __forceinline__ int router_segment_len(int H) {
    return (((H + ROUTER_SEGMENTS - 1) / ROUTER_SEGMENTS) + 3) & ~3;
}

__device__ __forceinline__ float router_segment_dot(const float* __restrict__ h, const float* __restrict__ w,
                                                    int begin, int end, bool vec, int lane) {
    float acc = 0.0f;
    if (end > begin) {
        if (vec) {
            const float4* h4 = reinterpret_cast<const float4*>(h + begin);
            const float4* w4 = reinterpret_cast<const float4*>(w + begin);
            const int n4 = (end - begin) >> 2;       // vec implies H % 4 == 0: every segment is whole pieces
#pragma unroll 8
            for (int i = lane; i < n4; i += 32) {
                const float4 a = h4[i], b = __ldg(w4 + i);
                acc = fmaf(a.x, b.x, acc);
                acc = fmaf(a.y, b.y, acc);
                acc = fmaf(a.z, b.z, acc);
                acc = fmaf(a.w, b.w, acc);
            }
        } else {
            for (int i = begin + lane; i < end; i += 32) acc = fmaf(h[i], w[i], acc);
        }
    }
    return warp_sum(acc);
}

__device__ __forceinline__ void router_pick(const float* r, int E, int* expert_id, float* expert_weight) {
    int best = 0;
    float best_p = 1.0f / (1.0f + expf(-r[0]));
    for (int e = 1; e < E; ++e) {
        const float p = 1.0f / (1.0f + expf(-r[e]));
        if (p > best_p) {
            best_p = p;
            best = e;
        }
    }
    *expert_id = best;
    *expert_weight = best_p;
}

// Many tokens: one block serves TPB consecutive tokens and its eight warps take one segment each, so a
// warp reads its slice of the activations from global memory (nobody else needs it) and its slice of a
// router row once for all the block's tokens; the experts go by in passes of EPP, TPB x EPP sums per lane.
// The segment sums meet in shared memory and are added in ascending order.
template <int TPB, int EPP>
__global__ void __launch_bounds__(ROUTER_SEGMENTS * 32)
router_top1_tiled_kernel(const float* __restrict__ h, const float* __restrict__ wr, int T, int H, int E,
                         int* __restrict__ expert_id, float* __restrict__ expert_weight,
                         float* __restrict__ logits_out) {
    extern __shared__ __align__(16) float smem[];
    float* seg_s = smem;                                  // [segments][TPB][E]
    float* r_s = smem + ROUTER_SEGMENTS * TPB * E;        // [TPB][E]
    const int t0 = blockIdx.x * TPB;
    const int n_tok = min(TPB, T - t0);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const bool vec = (H % 4 == 0) && ((reinterpret_cast<uintptr_t>(wr) & 15) == 0) &&
                     ((reinterpret_cast<uintptr_t>(h) & 15) == 0);
    const int seg = router_segment_len(H);
    const int begin = min(H, warp * seg), end = min(H, begin + seg);
    const float* hb = h + (size_t)t0 * H;
    for (int e0 = 0; e0 < E; e0 += EPP) {
        float acc[TPB][EPP];
#pragma unroll
        for (int tt = 0; tt < TPB; ++tt)
#pragma unroll
            for (int ee = 0; ee < EPP; ++ee) acc[tt][ee] = 0.0f;
        if (vec) {
            const int n4 = (end - begin) >> 2;
            for (int i = lane; i < n4; i += 32) {
                float4 a[TPB];
#pragma unroll
                for (int tt = 0; tt < TPB; ++tt)
                    a[tt] = (tt < n_tok) ? reinterpret_cast<const float4*>(hb + (size_t)tt * H + begin)[i]
                                         : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
                for (int ee = 0; ee < EPP; ++ee) {
                    if (e0 + ee < E) {
                        const float4 b = __ldg(reinterpret_cast<const float4*>(wr + (size_t)(e0 + ee) * H + begin) + i);
#pragma unroll
                        for (int tt = 0; tt < TPB; ++tt) {
                            acc[tt][ee] = fmaf(a[tt].x, b.x, acc[tt][ee]);
                            acc[tt][ee] = fmaf(a[tt].y, b.y, acc[tt][ee]);
                            acc[tt][ee] = fmaf(a[tt].z, b.z, acc[tt][ee]);
                            acc[tt][ee] = fmaf(a[tt].w, b.w, acc[tt][ee]);
                        }
                    }
                }
            }
        } else {
            for (int i = begin + lane; i < end; i += 32) {
                float a[TPB];
#pragma unroll
                for (int tt = 0; tt < TPB; ++tt) a[tt] = (tt < n_tok) ? hb[(size_t)tt * H + i] : 0.0f;
#pragma unroll
                for (int ee = 0; ee < EPP; ++ee) {
                    if (e0 + ee < E) {
                        const float b = wr[(size_t)(e0 + ee) * H + i];
#pragma unroll
                        for (int tt = 0; tt < TPB; ++tt) acc[tt][ee] = fmaf(a[tt], b, acc[tt][ee]);
                    }
                }
            }
        }
#pragma unroll
        for (int tt = 0; tt < TPB; ++tt)
#pragma unroll
            for (int ee = 0; ee < EPP; ++ee) {
                const float part = warp_sum(acc[tt][ee]);
                if (lane == 0 && e0 + ee < E) seg_s[(warp * TPB + tt) * E + e0 + ee] = part;
            }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < TPB * E; i += ROUTER_SEGMENTS * 32) {
        float total = 0.0f;
#pragma unroll
        for (int sgm = 0; sgm < ROUTER_SEGMENTS; ++sgm) total += seg_s[sgm * TPB * E + i];
        r_s[i] = total;
    }
    __syncthreads();
    if (logits_out)
        for (int i = threadIdx.x; i < n_tok * E; i += ROUTER_SEGMENTS * 32) logits_out[(size_t)t0 * E + i] = r_s[i];
    if (threadIdx.x < n_tok)
        router_pick(r_s + threadIdx.x * E, E, expert_id + t0 + threadIdx.x, expert_weight + t0 + threadIdx.x);
}

template <int TPB, int EPP>
static int launch_router(const float* h, const float* wr, int T, int H, int E, int* expert_id, float* expert_weight,
                         float* logits_out, cudaStream_t stream) {
    const size_t smem = (size_t)(ROUTER_SEGMENTS + 1) * TPB * E * sizeof(float);
    if (smem > 200 * 1024) return SHARPI_BAD_ARGUMENT;
    if (smem > 48 * 1024) {
        cudaError_t err = cudaFuncSetAttribute(router_top1_tiled_kernel<TPB, EPP>,
                                               cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (err != cudaSuccess) return SHARPI_LAUNCH_FAILED;
    }
    router_top1_tiled_kernel<TPB, EPP><<<(T + TPB - 1) / TPB, ROUTER_SEGMENTS * 32, smem, stream>>>(
        h, wr, T, H, E, expert_id, expert_weight, logits_out);
    SHARPI_CHECK_LAUNCH();
    return SHARPI_OK;
}

// Very many tokens (prompts): a warp keeps its segment of four router rows in registers and streams the
// block's tokens past them, so the router is read once per block of STREAM_TPB tokens and a token's loads do
// not wait for another token's.  NI = four-element pieces of a segment per lane (the width is at most
// 1024 * NI).  The sums are formed exactly as in router_segment_dot.
constexpr int STREAM_TPB = 16;
constexpr int STREAM_EPP = 4;

template <int NI>
__global__ void __launch_bounds__(ROUTER_SEGMENTS * 32)
router_top1_stream_kernel(const float* __restrict__ h, const float* __restrict__ wr, int T, int H, int E,
                          int* __restrict__ expert_id, float* __restrict__ expert_weight,
                          float* __restrict__ logits_out) {
    extern __shared__ __align__(16) float smem[];
    float* seg_s = smem;                                         // [segments][STREAM_TPB][E]
    float* r_s = smem + ROUTER_SEGMENTS * STREAM_TPB * E;        // [STREAM_TPB][E]
    const int t0 = blockIdx.x * STREAM_TPB;
    const int n_tok = min(STREAM_TPB, T - t0);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int seg = router_segment_len(H);
    const int begin = min(H, warp * seg), end = min(H, begin + seg);
    const int n4 = (end - begin) >> 2;                           // H % 4 == 0 here
    for (int e0 = 0; e0 < E; e0 += STREAM_EPP) {
        float4 b[STREAM_EPP][NI];
#pragma unroll
        for (int ee = 0; ee < STREAM_EPP; ++ee)
#pragma unroll
            for (int k = 0; k < NI; ++k) {
                const int i = lane + 32 * k;
                b[ee][k] = (e0 + ee < E && i < n4)
                               ? __ldg(reinterpret_cast<const float4*>(wr + (size_t)(e0 + ee) * H + begin) + i)
                               : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            }
#pragma unroll 2
        for (int tt = 0; tt < n_tok; ++tt) {
            const float4* a4 = reinterpret_cast<const float4*>(h + (size_t)(t0 + tt) * H + begin);
            float4 a[NI];
#pragma unroll
            for (int k = 0; k < NI; ++k) {
                const int i = lane + 32 * k;
                a[k] = i < n4 ? a4[i] : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            }
#pragma unroll
            for (int ee = 0; ee < STREAM_EPP; ++ee) {
                float acc = 0.0f;
#pragma unroll
                for (int k = 0; k < NI; ++k) {
                    if (lane + 32 * k < n4) {                    // a lane adds only the pieces it has, in order
                        acc = fmaf(a[k].x, b[ee][k].x, acc);
                        acc = fmaf(a[k].y, b[ee][k].y, acc);
                        acc = fmaf(a[k].z, b[ee][k].z, acc);
                        acc = fmaf(a[k].w, b[ee][k].w, acc);
                    }
                }
                const float part = warp_sum(acc);
                if (lane == 0 && e0 + ee < E) seg_s[(warp * STREAM_TPB + tt) * E + e0 + ee] = part;
            }
        }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < n_tok * E; i += ROUTER_SEGMENTS * 32) {
        float total = 0.0f;
#pragma unroll
        for (int sgm = 0; sgm < ROUTER_SEGMENTS; ++sgm) total += seg_s[sgm * STREAM_TPB * E + i];
        r_s[i] = total;
    }
    __syncthreads();
    if (logits_out)
        for (int i = threadIdx.x; i < n_tok * E; i += ROUTER_SEGMENTS * 32) logits_out[(size_t)t0 * E + i] = r_s[i];
    if (threadIdx.x < n_tok)
        router_pick(r_s + threadIdx.x * E, E, expert_id + t0 + threadIdx.x, expert_weight + t0 + threadIdx.x);
}

template <int NI>
static int launch_router_stream(const float* h, const float* wr, int T, int H, int E, int* expert_id,
                                float* expert_weight, float* logits_out, cudaStream_t stream) {
    const size_t smem = (size_t)(ROUTER_SEGMENTS + 1) * STREAM_TPB * E * sizeof(float);
    if (smem > 48 * 1024) {
        cudaError_t err = cudaFuncSetAttribute(router_top1_stream_kernel<NI>,
                                               cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (err != cudaSuccess) return SHARPI_LAUNCH_FAILED;
    }
    router_top1_stream_kernel<NI><<<(T + STREAM_TPB - 1) / STREAM_TPB, ROUTER_SEGMENTS * 32, smem, stream>>>(
        h, wr, T, H, E, expert_id, expert_weight, logits_out);
    SHARPI_CHECK_LAUNCH();
    return SHARPI_OK;
}

// Very many tokens, a row that fits shared memory: the block's SMEM_TPB tokens are brought into shared memory once
// and every pass of EPP router rows (held in registers, as above) runs over them there, so the activations
// cross into the SM once instead of once per pass (with 16 experts the kernel above reads them four times).
// The sums are formed exactly as in router_segment_dot.
constexpr int SMEM_TPB = 8;
constexpr int SMEM_SHARES = 1;      // warps per segment, each with every SMEM_SHARES-th token: more warps to hide latencies
constexpr int SMEM_THREADS = ROUTER_SEGMENTS * 32 * SMEM_SHARES;

template <int NI, int EPP>
__device__ __forceinline__ void router_rows_load(float4 (&b)[EPP][NI], const float* __restrict__ wr, int e0, int E,
                                                 int H, int begin, int n4, int lane) {
#pragma unroll
    for (int ee = 0; ee < EPP; ++ee)
#pragma unroll
        for (int k = 0; k < NI; ++k) {
            const int i = lane + 32 * k;
            b[ee][k] = (e0 + ee < E && i < n4)
                           ? __ldg(reinterpret_cast<const float4*>(wr + (size_t)(e0 + ee) * H + begin) + i)
                           : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        }
}

// Sums of NV values over the warp, each formed by the same tree of additions as warp_sum (partner 16, 8, 4, 2,
// 1 away; a + b is b + a), but halving the number of values a lane carries at each of the first steps instead of
// carrying all of them through five: 9 shuffles for eight values, not 40.  Lane l ends with the sum of value
// l >> (5 - log2 NV).
template <int NV>
__device__ __forceinline__ float warp_sums_scattered(float (&v)[NV], int lane) {
    int o = 16;
#pragma unroll
    for (int n = NV; n > 1; n >>= 1, o >>= 1) {
        const bool upper = (lane & o) != 0;
#pragma unroll
        for (int j = 0; j < n / 2; ++j) {
            const float mine = upper ? v[n / 2 + j] : v[j];
            const float theirs = upper ? v[j] : v[n / 2 + j];
            v[j] = mine + __shfl_xor_sync(0xffffffffu, theirs, o);
        }
    }
#pragma unroll
    for (; o > 0; o >>= 1) v[0] += __shfl_xor_sync(0xffffffffu, v[0], o);
    return v[0];
}

template <int NI, int EPP>
__device__ __forceinline__ void router_rows_apply(const float4 (&b)[EPP][NI], const float* h_s, float* seg_s, int e0,
                                                  int E, int H, int begin, int n4, int first, int n_tok, int warp,
                                                  int lane) {
    constexpr int NV = 2 * EPP, OWNERS = 32 / NV;                // two tokens at a time
    for (int tt = first; tt < n_tok; tt += 2 * SMEM_SHARES) {
        float v[NV];
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int t = min(tt + half * SMEM_SHARES, n_tok - 1);   // an odd last token is computed twice, stored once
            const float4* a4 = reinterpret_cast<const float4*>(h_s + (size_t)t * H + begin);
            float4 a[NI];
#pragma unroll
            for (int k = 0; k < NI; ++k) {
                const int i = lane + 32 * k;
                a[k] = i < n4 ? a4[i] : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            }
#pragma unroll
            for (int ee = 0; ee < EPP; ++ee) {
                float acc = 0.0f;
#pragma unroll
                for (int k = 0; k < NI; ++k) {
                    if (lane + 32 * k < n4) {                    // a lane adds only the pieces it has, in order
                        acc = fmaf(a[k].x, b[ee][k].x, acc);
                        acc = fmaf(a[k].y, b[ee][k].y, acc);
                        acc = fmaf(a[k].z, b[ee][k].z, acc);
                        acc = fmaf(a[k].w, b[ee][k].w, acc);
                    }
                }
                v[half * EPP + ee] = acc;
            }
        }
        const float part = warp_sums_scattered<NV>(v, lane);
        const int which = lane / OWNERS, t = tt + (which / EPP) * SMEM_SHARES, e = e0 + which % EPP;
        if (lane % OWNERS == 0 && t < n_tok && e < E) seg_s[(warp * SMEM_TPB + t) * E + e] = part;
    }
}

template <int NI, int EPP>
__global__ void __launch_bounds__(SMEM_THREADS)
router_top1_smem_kernel(const float* __restrict__ h, const float* __restrict__ wr, int T, int H, int E,
                        int* __restrict__ expert_id, float* __restrict__ expert_weight,
                        float* __restrict__ logits_out) {
    extern __shared__ __align__(16) float smem[];
    float* h_s = smem;                                           // [SMEM_TPB][H]
    float* seg_s = h_s + (size_t)SMEM_TPB * H;                   // [segments][SMEM_TPB][E]
    float* r_s = seg_s + ROUTER_SEGMENTS * SMEM_TPB * E;         // [SMEM_TPB][E]
    const int t0 = blockIdx.x * SMEM_TPB;
    const int n_tok = min(SMEM_TPB, T - t0);
    const int warp = (threadIdx.x >> 5) % ROUTER_SEGMENTS, share = (threadIdx.x >> 5) / ROUTER_SEGMENTS;
    const int lane = threadIdx.x & 31;
    {
        // Asynchronous 16-byte copies: all of a thread's pieces are in flight at once, so the tile arrives at the
        // rate the SM can take it instead of one memory latency per few pieces.  H % 4 == 0 here.
        const float* src = h + (size_t)t0 * H;
        const uint32_t dst = (uint32_t)__cvta_generic_to_shared(h_s);
        const int n = n_tok * (H >> 2);
        for (int i = threadIdx.x; i < n; i += SMEM_THREADS)
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst + 16u * i), "l"(src + 4 * (size_t)i)
                         : "memory");
        asm volatile("cp.async.commit_group;" ::: "memory");
    }
    const int seg = router_segment_len(H);
    const int begin = min(H, warp * seg), end = min(H, begin + seg);
    const int n4 = (end - begin) >> 2;
    float4 b[EPP][NI];
    for (int e0 = 0; e0 < E; e0 += EPP) {
        router_rows_load<NI, EPP>(b, wr, e0, E, H, begin, n4, lane);
        if (e0 == 0) {                                           // the first router rows are on their way by now
            asm volatile("cp.async.wait_group 0;" ::: "memory");
            __syncthreads();
        }
        router_rows_apply<NI, EPP>(b, h_s, seg_s, e0, E, H, begin, n4, share, n_tok, warp, lane);
    }
    __syncthreads();
    for (int i = threadIdx.x; i < n_tok * E; i += SMEM_THREADS) {
        float total = 0.0f;
#pragma unroll
        for (int sgm = 0; sgm < ROUTER_SEGMENTS; ++sgm) total += seg_s[sgm * SMEM_TPB * E + i];
        r_s[i] = total;
    }
    __syncthreads();
    if (logits_out)
        for (int i = threadIdx.x; i < n_tok * E; i += SMEM_THREADS) logits_out[(size_t)t0 * E + i] = r_s[i];
    if (threadIdx.x < n_tok)
        router_pick(r_s + threadIdx.x * E, E, expert_id + t0 + threadIdx.x, expert_weight + t0 + threadIdx.x);
}

static size_t router_smem_bytes(int H, int E) {
    return ((size_t)SMEM_TPB * H + (size_t)(ROUTER_SEGMENTS + 1) * SMEM_TPB * E) * sizeof(float);
}

template <int NI>
static int launch_router_smem(const float* h, const float* wr, int T, int H, int E, int* expert_id,
                              float* expert_weight, float* logits_out, cudaStream_t stream) {
    const size_t smem = router_smem_bytes(H, E);
    constexpr int EPP = NI <= 5 ? 8 : 4;                         // EPP x NI float4 of router rows in registers
    cudaError_t err = cudaFuncSetAttribute(router_top1_smem_kernel<NI, EPP>,
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (err != cudaSuccess) return SHARPI_LAUNCH_FAILED;
    router_top1_smem_kernel<NI, EPP><<<(T + SMEM_TPB - 1) / SMEM_TPB, SMEM_THREADS, smem, stream>>>(
        h, wr, T, H, E, expert_id, expert_weight, logits_out);
    SHARPI_CHECK_LAUNCH();
    return SHARPI_OK;
}

// Few tokens: what costs time is the chain of dependent loads of one block walking every expert, so each
// (token, expert) pair gets a block of its own whose eight warps take one segment each; every load of the
// step is then in flight at once.  The logits go to `logits`; the block that finishes last for a token (a
// ticket counter per token, which it resets) picks the expert.
__global__ void __launch_bounds__(ROUTER_SEGMENTS * 32)
router_top1_small_kernel(const float* __restrict__ h, const float* __restrict__ wr, int H, int E,
                         int* __restrict__ expert_id, float* __restrict__ expert_weight,
                         float* __restrict__ logits, int* __restrict__ tickets, int* __restrict__ offsets,
                         int* __restrict__ sorted_rows) {
    __shared__ float seg_s[ROUTER_SEGMENTS];
    __shared__ int last_s, sort_s;
    pdl_wait();
    const int t = blockIdx.x, e = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const bool vec = (H % 4 == 0) && ((reinterpret_cast<uintptr_t>(wr) & 15) == 0) &&
                     ((reinterpret_cast<uintptr_t>(h) & 15) == 0);
    const int seg = router_segment_len(H);
    const int begin = min(H, warp * seg), end = min(H, begin + seg);
    const float part = router_segment_dot(h + (size_t)t * H, wr + (size_t)e * H, begin, end, vec, lane);
    if (lane == 0) seg_s[warp] = part;
    __syncthreads();
    if (threadIdx.x == 0) {
        float total = 0.0f;
#pragma unroll
        for (int sgm = 0; sgm < ROUTER_SEGMENTS; ++sgm) total += seg_s[sgm];
        logits[(size_t)t * E + e] = total;
        __threadfence();
        last_s = (atomicAdd(&tickets[t], 1) == (int)gridDim.y - 1);
        if (last_s) {
            tickets[t] = 0;
            __threadfence();
            const float* r = logits + (size_t)t * E;
            int best = 0;
            float best_p = 1.0f / (1.0f + expf(-__ldcg(r)));
            for (int x = 1; x < E; ++x) {
                const float p = 1.0f / (1.0f + expf(-__ldcg(r + x)));
                if (p > best_p) {
                    best_p = p;
                    best = x;
                }
            }
            expert_id[t] = best;
            expert_weight[t] = best_p;
        }
    }
    if (!sorted_rows) return;
    // The block that picks the step's last expert also sorts the step's (at most 32) rows by expert: a second
    // ticket counts the tokens that have theirs.  The same stable counting sort as moe_sort_kernel.
    if (threadIdx.x == 0) {
        sort_s = 0;
        if (last_s) {
            __threadfence();
            sort_s = (atomicAdd(&tickets[32], 1) == (int)gridDim.x - 1);
            if (sort_s) tickets[32] = 0;
        }
    }
    __syncthreads();
    if (!sort_s || warp != 0) return;
    __threadfence();
    const int T = gridDim.x;
    const int id = (lane < T) ? __ldcg(expert_id + lane) : -1;
    const unsigned lt = (1u << lane) - 1u;
    int run = 0;
    for (int x = 0; x < E; ++x) {
        const unsigned mask = __ballot_sync(0xffffffffu, id == x);
        if (lane == 0) offsets[x] = run;
        if (id == x) sorted_rows[run + __popc(mask & lt)] = lane;
        run += __popc(mask);
    }
    if (lane == 0) offsets[E] = run;
}

static int launch_sort(const int* expert_id, int T, int E, int* offsets, int* sorted_rows, cudaStream_t stream);

// `scratch`, optional: [32 * E] floats then [33] zero-initialised ints (the tickets, left zero again).
// With it, steps of up to 32 tokens take the kernel that gives every (token, expert) pair a block.
// `offsets` [E + 1] and `sorted_rows` [T], optional (both or none): the rows sorted by expert as sharpi_moe_sort
// gives them, from the same launch when the step is small, from a second one otherwise.
SHARPI_API int sharpi_router_top1(const float* h, const float* wr, int T, int H, int E, int gate, int* expert_id,
                                  float* expert_weight, float* logits_out, void* scratch, int* offsets,
                                  int* sorted_rows, cudaStream_t stream) {
    if ((offsets == nullptr) != (sorted_rows == nullptr)) return SHARPI_BAD_ARGUMENT;
    if (T <= 0) return offsets ? launch_sort(expert_id, 0, E, offsets, sorted_rows, stream) : SHARPI_OK;
    if (H <= 0 || E <= 0 || gate != ROUTER_GATE_SIGMOID) return SHARPI_BAD_ARGUMENT;
    if (T <= 32 && scratch && E <= 65535) {
        float* logits = logits_out ? logits_out : reinterpret_cast<float*>(scratch);
        int* tickets = reinterpret_cast<int*>(reinterpret_cast<float*>(scratch) + (size_t)32 * E);
        SHARPI_LAUNCH_PDL(router_top1_small_kernel, dim3(T, E), ROUTER_SEGMENTS * 32, 0, stream, h, wr, H, E, expert_id,
                          expert_weight, logits, tickets, offsets, sorted_rows);
        return SHARPI_OK;
    }
    // many tokens: eight share a block and its reads of the router rows (four with sixteen experts to a pass
    // measured slower: the rows are re-read from L2 once per block); fewer: two, for more blocks
    int rc;
    const bool vec = (H % 4 == 0) && ((reinterpret_cast<uintptr_t>(wr) & 15) == 0) &&
                     ((reinterpret_cast<uintptr_t>(h) & 15) == 0);
    const int pieces = (router_segment_len(H) / 4 + 31) / 32;          // per lane and segment
    if (T >= 1024 && vec && pieces <= 8 && router_smem_bytes(H, E) <= 200 * 1024) {
        switch (pieces) {
            case 1: rc = launch_router_smem<1>(h, wr, T, H, E, expert_id, expert_weight, logits_out, stream); break;
            case 2: rc = launch_router_smem<2>(h, wr, T, H, E, expert_id, expert_weight, logits_out, stream); break;
            case 3: rc = launch_router_smem<3>(h, wr, T, H, E, expert_id, expert_weight, logits_out, stream); break;
            case 4: rc = launch_router_smem<4>(h, wr, T, H, E, expert_id, expert_weight, logits_out, stream); break;
            case 5: rc = launch_router_smem<5>(h, wr, T, H, E, expert_id, expert_weight, logits_out, stream); break;
            case 6: rc = launch_router_smem<6>(h, wr, T, H, E, expert_id, expert_weight, logits_out, stream); break;
            case 7: rc = launch_router_smem<7>(h, wr, T, H, E, expert_id, expert_weight, logits_out, stream); break;
            default: rc = launch_router_smem<8>(h, wr, T, H, E, expert_id, expert_weight, logits_out, stream); break;
        }
    } else if (T >= 1024 && vec && pieces <= 8 && (size_t)(ROUTER_SEGMENTS + 1) * STREAM_TPB * E * sizeof(float) <= 200 * 1024) {
        switch (pieces) {
            case 1: rc = launch_router_stream<1>(h, wr, T, H, E, expert_id, expert_weight, logits_out, stream); break;
            case 2: rc = launch_router_stream<2>(h, wr, T, H, E, expert_id, expert_weight, logits_out, stream); break;
            case 3: rc = launch_router_stream<3>(h, wr, T, H, E, expert_id, expert_weight, logits_out, stream); break;
            case 4: rc = launch_router_stream<4>(h, wr, T, H, E, expert_id, expert_weight, logits_out, stream); break;
            case 5: rc = launch_router_stream<5>(h, wr, T, H, E, expert_id, expert_weight, logits_out, stream); break;
            case 6: rc = launch_router_stream<6>(h, wr, T, H, E, expert_id, expert_weight, logits_out, stream); break;
            case 7: rc = launch_router_stream<7>(h, wr, T, H, E, expert_id, expert_weight, logits_out, stream); break;
            default: rc = launch_router_stream<8>(h, wr, T, H, E, expert_id, expert_weight, logits_out, stream); break;
        }
    } else if (T >= 1024 && (size_t)(ROUTER_SEGMENTS + 1) * 8 * E * sizeof(float) <= 200 * 1024)
        rc = launch_router<8, 4>(h, wr, T, H, E, expert_id, expert_weight, logits_out, stream);
    else
        rc = launch_router<2, 8>(h, wr, T, H, E, expert_id, expert_weight, logits_out, stream);
    if (rc != SHARPI_OK || !offsets) return rc;
    return launch_sort(expert_id, T, E, offsets, sorted_rows, stream);
}

// ---------------------------------------------------------------------------------------
// Stable counting sort of the rows by expert, in one block: offsets[e] = first sorted row of
// expert e (offsets[E] = T), sorted_rows[r] = the row that stands at sorted position r.  Rows
// of one expert keep their order.  Warp w owns experts w, w + 32, ...: it walks all rows with
// ballots, once to count and once to place.
// ---------------------------------------------------------------------------------------
constexpr int SORT_THREADS = 1024;
constexpr int SORT_MAX_E = 1024;
constexpr int SORT_CHUNK = 4096;      // expert ids staged in shared memory at a time

__global__ void __launch_bounds__(SORT_THREADS)
moe_sort_kernel(const int* __restrict__ expert_id, int T, int E, int* __restrict__ offsets,
                int* __restrict__ sorted_rows) {
    __shared__ int cnt_s[SORT_MAX_E + 1];
    __shared__ int ids_s[SORT_CHUNK];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const unsigned lt = (1u << lane) - 1u;
    for (int e = threadIdx.x; e <= E; e += SORT_THREADS) cnt_s[e] = 0;
    for (int c0 = 0; c0 < T; c0 += SORT_CHUNK) {
        const int n_c = min(SORT_CHUNK, T - c0);
        __syncthreads();
        for (int i = threadIdx.x; i < n_c; i += SORT_THREADS) ids_s[i] = expert_id[c0 + i];
        __syncthreads();
        for (int e = warp; e < E; e += SORT_THREADS / 32) {
            int n = 0;
            for (int base = 0; base < n_c; base += 32) {
                const int t = base + lane;
                const bool mine = (t < n_c) && (ids_s[t] == e);
                n += __popc(__ballot_sync(0xffffffffu, mine));
            }
            if (lane == 0) cnt_s[e] += n;         // expert e belongs to this warp alone
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int run = 0;
        for (int e = 0; e < E; ++e) {
            const int n = cnt_s[e];
            cnt_s[e] = run;
            offsets[e] = run;
            run += n;
        }
        cnt_s[E] = run;
        offsets[E] = run;
    }
    for (int c0 = 0; c0 < T; c0 += SORT_CHUNK) {
        const int n_c = min(SORT_CHUNK, T - c0);
        __syncthreads();
        for (int i = threadIdx.x; i < n_c; i += SORT_THREADS) ids_s[i] = expert_id[c0 + i];
        __syncthreads();
        for (int e = warp; e < E; e += SORT_THREADS / 32) {
            int cursor = cnt_s[e];
            for (int base = 0; base < n_c; base += 32) {
                const int t = base + lane;
                const bool mine = (t < n_c) && (ids_s[t] == e);
                const unsigned mask = __ballot_sync(0xffffffffu, mine);
                if (mine) sorted_rows[cursor + __popc(mask & lt)] = c0 + t;
                cursor += __popc(mask);
            }
            if (lane == 0) cnt_s[e] = cursor;
        }
    }
}

static int launch_sort(const int* expert_id, int T, int E, int* offsets, int* sorted_rows, cudaStream_t stream) {
    if (E <= 0 || E > SORT_MAX_E || T < 0) return SHARPI_BAD_ARGUMENT;
    moe_sort_kernel<<<1, SORT_THREADS, 0, stream>>>(expert_id, T, E, offsets, sorted_rows);
    SHARPI_CHECK_LAUNCH();
    return SHARPI_OK;
}

SHARPI_API int sharpi_moe_sort(const int* expert_id, int T, int E, int* offsets, int* sorted_rows,
                               cudaStream_t stream) {
    return launch_sort(expert_id, T, E, offsets, sorted_rows, stream);
}
