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

constexpr int ROUTER_THREADS = 256;

// One block serves TPB consecutive tokens: a warp reads a router row once and forms the dot product
// with each of the block's tokens.  Every token's sum is the same chain of operations whatever TPB
// is (a lane adds its own stride-32 elements in order, the warp adds the 32 lane sums in a fixed
// tree), so the logits do not depend on how many tokens share a block.
template <int TPB>
__global__ void router_top1_kernel(const float* __restrict__ h, const float* __restrict__ wr, int T, int H, int E,
                                   int* __restrict__ expert_id, float* __restrict__ expert_weight,
                                   float* __restrict__ logits_out) {
    extern __shared__ __align__(16) float smem[];
    float* h_s = smem;                // [TPB][H]
    float* r_s = smem + TPB * H;      // [TPB][E]
    const int t0 = blockIdx.x * TPB;
    const int n_tok = min(TPB, T - t0);
    for (int i = threadIdx.x; i < TPB * H; i += ROUTER_THREADS) {
        const int tt = i / H;
        h_s[i] = (tt < n_tok) ? h[(size_t)t0 * H + i] : 0.0f;
    }
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const bool vec = (H % 4 == 0) && ((reinterpret_cast<uintptr_t>(wr) & 15) == 0);
    for (int e = warp; e < E; e += ROUTER_THREADS / 32) {
        const float* w = wr + (size_t)e * H;
        float acc[TPB];
#pragma unroll
        for (int tt = 0; tt < TPB; ++tt) acc[tt] = 0.0f;
        if (vec) {
            const float4* w4 = reinterpret_cast<const float4*>(w);
#pragma unroll 2
            for (int i = lane; i < H / 4; i += 32) {
                const float4 b = __ldg(w4 + i);
#pragma unroll
                for (int tt = 0; tt < TPB; ++tt) {
                    const float4 a = reinterpret_cast<const float4*>(h_s + tt * H)[i];
                    acc[tt] = fmaf(a.x, b.x, acc[tt]);
                    acc[tt] = fmaf(a.y, b.y, acc[tt]);
                    acc[tt] = fmaf(a.z, b.z, acc[tt]);
                    acc[tt] = fmaf(a.w, b.w, acc[tt]);
                }
            }
        } else {
            for (int i = lane; i < H; i += 32) {
                const float b = w[i];
#pragma unroll
                for (int tt = 0; tt < TPB; ++tt) acc[tt] = fmaf(h_s[tt * H + i], b, acc[tt]);
            }
        }
#pragma unroll
        for (int tt = 0; tt < TPB; ++tt) {
            const float total = warp_sum(acc[tt]);
            if (lane == 0) r_s[tt * E + e] = total;
        }
    }
    __syncthreads();
    if (logits_out)
        for (int i = threadIdx.x; i < n_tok * E; i += ROUTER_THREADS) logits_out[(size_t)t0 * E + i] = r_s[i];
    if (threadIdx.x < n_tok) {
        const float* r = r_s + threadIdx.x * E;
        int best = 0;
        float best_p = 1.0f / (1.0f + expf(-r[0]));
        for (int e = 1; e < E; ++e) {
            const float p = 1.0f / (1.0f + expf(-r[e]));
            if (p > best_p) {
                best_p = p;
                best = e;
            }
        }
        expert_id[t0 + threadIdx.x] = best;
        expert_weight[t0 + threadIdx.x] = best_p;
    }
}

template <int TPB>
static int launch_router(const float* h, const float* wr, int T, int H, int E, int* expert_id, float* expert_weight,
                         float* logits_out, cudaStream_t stream) {
    const size_t smem = (size_t)TPB * (H + E) * sizeof(float);
    if (smem > 200 * 1024) return SHARPI_BAD_ARGUMENT;
    if (smem > 48 * 1024) {
        cudaError_t err = cudaFuncSetAttribute(router_top1_kernel<TPB>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                               (int)smem);
        if (err != cudaSuccess) return SHARPI_LAUNCH_FAILED;
    }
    router_top1_kernel<TPB><<<(T + TPB - 1) / TPB, ROUTER_THREADS, smem, stream>>>(h, wr, T, H, E, expert_id,
                                                                                   expert_weight, logits_out);
    SHARPI_CHECK_LAUNCH();
    return SHARPI_OK;
}

SHARPI_API int sharpi_router_top1(const float* h, const float* wr, int T, int H, int E, int gate, int* expert_id,
                                  float* expert_weight, float* logits_out, cudaStream_t stream) {
    if (T <= 0) return SHARPI_OK;
    if (H <= 0 || E <= 0 || gate != ROUTER_GATE_SIGMOID) return SHARPI_BAD_ARGUMENT;
    // many tokens: four share a block and a read of the router; few tokens: one block each
    if (T >= 256 && (size_t)4 * (H + E) * sizeof(float) <= 200 * 1024)
        return launch_router<4>(h, wr, T, H, E, expert_id, expert_weight, logits_out, stream);
    return launch_router<1>(h, wr, T, H, E, expert_id, expert_weight, logits_out, stream);
}

// ---------------------------------------------------------------------------------------
// Stable counting sort of the rows by expert, in one block: offsets[e] = first sorted row of
// expert e (offsets[E] = T), sorted_rows[r] = the row that stands at sorted position r.  Rows
// of one expert keep their order.  Warp w owns experts w, w + 32, ...: it walks all rows with
// ballots, once to count and once to place.
// ---------------------------------------------------------------------------------------
constexpr int SORT_THREADS = 1024;
constexpr int SORT_MAX_E = 1024;

__global__ void moe_sort_kernel(const int* __restrict__ expert_id, int T, int E, int* __restrict__ offsets,
                                int* __restrict__ sorted_rows) {
    __shared__ int cnt_s[SORT_MAX_E + 1];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const unsigned lt = (1u << lane) - 1u;
    for (int e = warp; e < E; e += SORT_THREADS / 32) {
        int n = 0;
        for (int base = 0; base < T; base += 32) {
            const int t = base + lane;
            const bool mine = (t < T) && (expert_id[t] == e);
            n += __popc(__ballot_sync(0xffffffffu, mine));
        }
        if (lane == 0) cnt_s[e] = n;
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
    __syncthreads();
    for (int e = warp; e < E; e += SORT_THREADS / 32) {
        int cursor = cnt_s[e];
        for (int base = 0; base < T; base += 32) {
            const int t = base + lane;
            const bool mine = (t < T) && (expert_id[t] == e);
            const unsigned mask = __ballot_sync(0xffffffffu, mine);
            if (mine) sorted_rows[cursor + __popc(mask & lt)] = t;
            cursor += __popc(mask);
        }
    }
}

SHARPI_API int sharpi_moe_sort(const int* expert_id, int T, int E, int* offsets, int* sorted_rows,
                               cudaStream_t stream) {
    if (E <= 0 || E > SORT_MAX_E || T < 0) return SHARPI_BAD_ARGUMENT;
    moe_sort_kernel<<<1, SORT_THREADS, 0, stream>>>(expert_id, T, E, offsets, sorted_rows);
    SHARPI_CHECK_LAUNCH();
    return SHARPI_OK;
}
