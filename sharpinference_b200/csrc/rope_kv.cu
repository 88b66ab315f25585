// What happens to a fused Q|K|V projection before attention, in one pass over it:
// rotary position encoding of q and k, weightless L2 norm of q and k per head, the
// attention-temperature factor on q, the store of q for the attention kernel and the
// scatter of k and v into the pages of the cache.
//
// Reference order: RoPE, then the L2 norm, then the cache append
// (src/SharpInference.Engine/ForwardPass.cs:1635-1669); its CUDA path runs
// llm_rope_interleaved, llm_head_norm_pure and llm_kv_append one after the other
// (src/SharpInference.Cuda/CudaTextKernels.cs:653, :263, :850).  The temperature factor is
// not in the reference: q *= 1 + attn_scale * ln(1 + floor((pos + 1) / floor_scale)).
//
// Angles (pos * inv_freq), sin/cos, the norm's mean of squares and the temperature factor
// are fp32.  One warp owns one head of one token, so no result depends on the batch.  Head sizes
// that are multiples of four with interleaved pairs (or no rotation) take the kernel in which a lane
// owns whole 16-byte pieces, two pairs each; the others take the element-wise one.  Which of the two
// runs depends on the head size and the pairing alone.
#include "common.cuh"

enum RopePairing : int {
    ROPE_NONE = 0,
    ROPE_INTERLEAVED = 1,  // pairs (2j, 2j+1)
    ROPE_HALVES = 2,       // pairs (j, j + d/2)
};

struct QkvPostArgs {
    const float* qkv;        // [T, (nq + 2 nkv) * d]
    const int* positions;    // [T]
    const int* row_req;      // [T] index of the row's request in this step
    const int* block_table;  // [B, max_blocks] page ids of this layer's cache group
    const float* inv_freq;   // [d/2] or null
    void* q_out;             // [T, nq, d]
    void* kv_base;           // this layer's pages: [page][2][nkv][page_size][d]
    int T, nq, nkv, d;
    int max_blocks, page_size;
    int pairing;
    float l2_eps;            // < 0: no norm
    float temp_attn_scale;   // temperature factor on q; floor_scale <= 0: none
    float temp_floor_scale;
    int write_kv;            // 0: this layer reads a cache that another layer writes
};

template <typename TO>
__global__ void qkv_post_kernel(QkvPostArgs a) {
    const int warps_per_block = blockDim.x >> 5;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int slots = a.nq + 2 * a.nkv;
    const long long work = (long long)blockIdx.x * warps_per_block + warp;
    if (work >= (long long)a.T * slots) return;
    const int t = (int)(work / slots);
    const int slot = (int)(work % slots);
    const int d = a.d, half = d >> 1;
    const int pos = a.positions[t];
    const float* src = a.qkv + (size_t)t * slots * d + (size_t)slot * d;

    const bool is_q = slot < a.nq;
    const bool is_k = !is_q && slot < a.nq + a.nkv;
    const bool is_v = !is_q && !is_k;

    TO* dst;
    if (is_q) {
        dst = (TO*)a.q_out + ((size_t)t * a.nq + slot) * d;
    } else {
        if (!a.write_kv) return;
        const int head = is_k ? slot - a.nq : slot - a.nq - a.nkv;
        const int page = a.block_table[(size_t)a.row_req[t] * a.max_blocks + pos / a.page_size];
        if (page < 0) return;  // the host checks before the launch that every written position has a page
        const size_t plane = (size_t)a.nkv * a.page_size * d;
        dst = (TO*)a.kv_base + ((size_t)page * 2 + (is_k ? 0 : 1)) * plane +
              ((size_t)head * a.page_size + (pos % a.page_size)) * d;
    }

    if (is_v) {
        for (int i = lane; i < d; i += 32) dst[i] = from_float<TO>(src[i]);
        return;
    }

    // q or k: rotate, norm, scale.  A lane keeps its pairs in registers: up to 8 pairs per
    // lane covers head sizes up to 512.
    constexpr int MAX_PAIRS = 8;
    float x0[MAX_PAIRS], x1[MAX_PAIRS];
    float ss = 0.0f;
#pragma unroll
    for (int r = 0; r < MAX_PAIRS; ++r) {
        const int j = lane + 32 * r;
        if (j < half) {
            const int i0 = (a.pairing == ROPE_HALVES) ? j : 2 * j;
            const int i1 = (a.pairing == ROPE_HALVES) ? j + half : 2 * j + 1;
            float v0 = src[i0], v1 = src[i1];
            if (a.pairing != ROPE_NONE && a.inv_freq) {
                const float angle = (float)pos * a.inv_freq[j];
                float sn, cs;
                sincosf(angle, &sn, &cs);
                const float r0 = v0 * cs - v1 * sn;
                const float r1 = v0 * sn + v1 * cs;
                v0 = r0;
                v1 = r1;
            }
            x0[r] = v0;
            x1[r] = v1;
            ss += v0 * v0 + v1 * v1;
        } else {
            x0[r] = 0.0f;
            x1[r] = 0.0f;
        }
    }
    float scale = 1.0f;
    if (a.l2_eps >= 0.0f) {
        ss = warp_sum(ss);
        scale = 1.0f / sqrtf(ss / (float)d + a.l2_eps);
    }
    if (is_q && a.temp_floor_scale > 0.0f) {
        const float steps = floorf(((float)pos + 1.0f) / a.temp_floor_scale);
        scale *= 1.0f + a.temp_attn_scale * log1pf(steps);
    }
#pragma unroll
    for (int r = 0; r < MAX_PAIRS; ++r) {
        const int j = lane + 32 * r;
        if (j < half) {
            const int i0 = (a.pairing == ROPE_HALVES) ? j : 2 * j;
            const int i1 = (a.pairing == ROPE_HALVES) ? j + half : 2 * j + 1;
            dst[i0] = from_float<TO>(x0[r] * scale);
            dst[i1] = from_float<TO>(x1[r] * scale);
        }
    }
}

template <typename TO>
__device__ __forceinline__ void store4(TO* dst, float4 v);
template <>
__device__ __forceinline__ void store4<float>(float* dst, float4 v) {
    *reinterpret_cast<float4*>(dst) = v;
}
template <>
__device__ __forceinline__ void store4<bf16>(bf16* dst, float4 v) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
    uint2 w;
    w.x = *reinterpret_cast<uint32_t*>(&lo);
    w.y = *reinterpret_cast<uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(dst) = w;
}

// d % 4 == 0, pairs (2j, 2j+1) or no rotation: lane l owns the four-element pieces l, l + 32, ... of a head.
// A warp serves QKV_SLOTS consecutive heads (q, k or v) of one token: their loads are issued together, and
// the sines and cosines of the lane's pairs, which depend on the token alone, are taken once.
constexpr int QKV_SLOTS = 4;

template <typename TO, int MAX_PIECES>      // MAX_PIECES * 128 >= head size
__global__ void __launch_bounds__(256) qkv_post_vec_kernel(QkvPostArgs a) {
    pdl_wait();
    const int warps_per_block = blockDim.x >> 5;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int slots = a.nq + 2 * a.nkv;
    const int groups = (slots + QKV_SLOTS - 1) / QKV_SLOTS;
    const long long work = (long long)blockIdx.x * warps_per_block + warp;
    if (work >= (long long)a.T * groups) return;
    const int t = (int)(work / groups);
    const int slot0 = (int)(work % groups) * QKV_SLOTS;
    const int d = a.d, n4 = d >> 2;
    float4 x[QKV_SLOTS][MAX_PIECES];
#pragma unroll
    for (int s = 0; s < QKV_SLOTS; ++s) {
        const float4* __restrict__ src =
            reinterpret_cast<const float4*>(a.qkv + (size_t)t * slots * d + (size_t)(slot0 + s) * d);
#pragma unroll
        for (int r = 0; r < MAX_PIECES; ++r) {
            const int i = lane + 32 * r;
            x[s][r] = (slot0 + s < slots && i < n4) ? src[i] : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        }
    }
    const int pos = a.positions[t];
    const bool rotate = a.pairing != ROPE_NONE && a.inv_freq;
    float cs0[MAX_PIECES], sn0[MAX_PIECES], cs1[MAX_PIECES], sn1[MAX_PIECES];
    if (rotate && slot0 < a.nq + a.nkv) {               // the group holds at least one q or k head
#pragma unroll
        for (int r = 0; r < MAX_PIECES; ++r) {
            const int i = lane + 32 * r;
            if (i < n4) {
                const float2 f = __ldg(reinterpret_cast<const float2*>(a.inv_freq) + i);   // pairs 2i, 2i + 1
                sincosf((float)pos * f.x, &sn0[r], &cs0[r]);
                sincosf((float)pos * f.y, &sn1[r], &cs1[r]);
            }
        }
    }
    // where this token's keys and values go
    int page = -1;
    if (a.write_kv && slot0 + QKV_SLOTS > a.nq)
        page = a.block_table[(size_t)a.row_req[t] * a.max_blocks + pos / a.page_size];
    const size_t plane = (size_t)a.nkv * a.page_size * d;
    float temp = 1.0f;
    if (a.temp_floor_scale > 0.0f && slot0 < a.nq) {
        const float steps = floorf(((float)pos + 1.0f) / a.temp_floor_scale);
        temp = 1.0f + a.temp_attn_scale * log1pf(steps);
    }
#pragma unroll
    for (int s = 0; s < QKV_SLOTS; ++s) {
        const int slot = slot0 + s;
        if (slot >= slots) break;
        const bool is_q = slot < a.nq;
        const bool is_k = !is_q && slot < a.nq + a.nkv;
        TO* dst;
        if (is_q) {
            dst = (TO*)a.q_out + ((size_t)t * a.nq + slot) * d;
        } else {
            if (page < 0) continue;      // no cache write for this layer (the host checks that written positions have pages)
            const int head = is_k ? slot - a.nq : slot - a.nq - a.nkv;
            dst = (TO*)a.kv_base + ((size_t)page * 2 + (is_k ? 0 : 1)) * plane +
                  ((size_t)head * a.page_size + (pos % a.page_size)) * d;
        }
        float scale = 1.0f;
        if (is_q || is_k) {
            float ss = 0.0f;
#pragma unroll
            for (int r = 0; r < MAX_PIECES; ++r) {
                const int i = lane + 32 * r;
                if (i < n4) {
                    if (rotate) {
                        const float4 v = x[s][r];
                        x[s][r] = make_float4(v.x * cs0[r] - v.y * sn0[r], v.x * sn0[r] + v.y * cs0[r],
                                              v.z * cs1[r] - v.w * sn1[r], v.z * sn1[r] + v.w * cs1[r]);
                    }
                    ss += x[s][r].x * x[s][r].x + x[s][r].y * x[s][r].y;
                    ss += x[s][r].z * x[s][r].z + x[s][r].w * x[s][r].w;
                }
            }
            if (a.l2_eps >= 0.0f) {
                ss = warp_sum(ss);
                scale = 1.0f / sqrtf(ss / (float)d + a.l2_eps);
            }
            if (is_q) scale *= temp;
        }
#pragma unroll
        for (int r = 0; r < MAX_PIECES; ++r) {
            const int i = lane + 32 * r;
            if (i < n4)
                store4<TO>(dst + 4 * i, make_float4(x[s][r].x * scale, x[s][r].y * scale, x[s][r].z * scale, x[s][r].w * scale));
        }
    }
}

SHARPI_API int sharpi_qkv_post(const float* qkv, const int* positions, const int* row_req, const int* block_table,
                               const float* inv_freq, void* q_out, void* kv_base, int out_dtype, int T, int nq,
                               int nkv, int d, int max_blocks, int page_size, int pairing, float l2_eps,
                               float temp_attn_scale, float temp_floor_scale, int write_kv,
                               cudaStream_t stream) {
    if (T <= 0) return SHARPI_OK;
    if (nq <= 0 || nkv <= 0 || d <= 0 || (d & 1) || d > 512 || page_size <= 0 || max_blocks <= 0)
        return SHARPI_BAD_ARGUMENT;
    if (pairing != ROPE_NONE && pairing != ROPE_INTERLEAVED && pairing != ROPE_HALVES) return SHARPI_BAD_ARGUMENT;
    QkvPostArgs a;
    a.qkv = qkv; a.positions = positions; a.row_req = row_req; a.block_table = block_table;
    a.inv_freq = inv_freq; a.q_out = q_out; a.kv_base = kv_base;
    a.T = T; a.nq = nq; a.nkv = nkv; a.d = d; a.max_blocks = max_blocks; a.page_size = page_size;
    a.pairing = inv_freq ? pairing : ROPE_NONE; a.l2_eps = l2_eps;
    a.temp_attn_scale = temp_attn_scale; a.temp_floor_scale = temp_floor_scale; a.write_kv = write_kv;
    if (out_dtype != SHARPI_F32 && out_dtype != SHARPI_BF16) return SHARPI_BAD_ARGUMENT;
    const long long work = (long long)T * (nq + 2 * nkv);
    const long long vec_work = (long long)T * ((nq + 2 * nkv + QKV_SLOTS - 1) / QKV_SLOTS);
    const uintptr_t ptrs = reinterpret_cast<uintptr_t>(qkv) | reinterpret_cast<uintptr_t>(q_out) |
                           reinterpret_cast<uintptr_t>(kv_base) | reinterpret_cast<uintptr_t>(inv_freq);
    if (d % 4 == 0 && a.pairing != ROPE_HALVES && (ptrs & 15) == 0) {
        const int warps = 8;
        const long long blocks = (vec_work + warps - 1) / warps;
        if (blocks > 2147483647LL) return SHARPI_BAD_ARGUMENT;
#define QKV_CASE(TO, P)                                                                     \
    do {                                                                                    \
        auto kern = qkv_post_vec_kernel<TO, P>;                                             \
        SHARPI_LAUNCH_PDL(kern, (unsigned)blocks, warps * 32, 0, stream, a);                \
    } while (0)
        if (out_dtype == SHARPI_F32) {
            if (d <= 128) QKV_CASE(float, 1); else if (d <= 256) QKV_CASE(float, 2); else QKV_CASE(float, 4);
        } else {
            if (d <= 128) QKV_CASE(bf16, 1); else if (d <= 256) QKV_CASE(bf16, 2); else QKV_CASE(bf16, 4);
        }
#undef QKV_CASE
        return SHARPI_OK;
    }
    const int warps = 4;
    const long long blocks = (work + warps - 1) / warps;
    if (blocks > 2147483647LL) return SHARPI_BAD_ARGUMENT;
    if (out_dtype == SHARPI_F32)
        qkv_post_kernel<float><<<(unsigned)blocks, warps * 32, 0, stream>>>(a);
    else if (out_dtype == SHARPI_BF16)
        qkv_post_kernel<bf16><<<(unsigned)blocks, warps * 32, 0, stream>>>(a);
    else
        return SHARPI_BAD_ARGUMENT;
    SHARPI_CHECK_LAUNCH();
    return SHARPI_OK;
}
