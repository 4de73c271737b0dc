// Gated GQA decode attention over a paged KV cache: per-head RMSNorm of q and k, partial RoPE on
// dims 0..63 (pairs i, i+32), KV append, f32 scores and softmax, bf16 softmax weights, P.V, and
// the sigmoid output gate, in one kernel.
//
// One CTA per (row, kv head): the 4 query heads that share a KV head are processed together so
// every cached K and V row is read from HBM once per row.  A warp reads a whole 512-byte K (or V)
// row with 16-byte loads; the cache is addressed through a per-lane page table
// (page = 64 positions x 2 kv heads x 256 dims).
//
// Replaces attn_decode_layer / mtp_attn_row (engine/kernels.h:730-906,
// engine/kernels_attn.cpp:995-1068); arithmetic follows speccheck/specimpl.py:320-397 as executed,
// except that cached keys are bf16 (the engine's cache dtype, engine/state.h:90).
#include "q35_common.cuh"

namespace q35 {

constexpr int kAttnMaxCtx = 8192;
constexpr int kOffK = 4096, kOffV = 4608;

__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
    f[0] = lo_bf(v.x); f[1] = hi_bf(v.x); f[2] = lo_bf(v.y); f[3] = hi_bf(v.y);
    f[4] = lo_bf(v.z); f[5] = hi_bf(v.z); f[6] = lo_bf(v.w); f[7] = hi_bf(v.w);
}

// Zero-centred RMSNorm of one 256-wide head held 8 values per lane, then partial RoPE.
// Returns the f32 result in x (rotated dims are NOT rounded; un-rotated dims are bf16 values).
__device__ __forceinline__ void head_norm_rope(float (&x)[8], const uint16_t* __restrict__ w, int ln,
                                               int rope_pos, const float* __restrict__ inv_freq) {
    float ss = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) ss += x[e] * x[e];
    ss = warp_sum(ss);
    const float inv = rsqrt_acc(ss * (1.0f / kHeadDim) + kEps);
    const uint4 wv = *reinterpret_cast<const uint4*>(w + 8 * ln);
    float wf[8];
    unpack8(wv, wf);
#pragma unroll
    for (int e = 0; e < 8; ++e) x[e] = bfround(__fmul_rn(__fmul_rn(x[e], inv), 1.0f + wf[e]));
    // lanes 0..3 hold dims 0..31, lanes 4..7 hold dims 32..63; partner of dim d is d ^ 32
#pragma unroll
    for (int e = 0; e < 8; ++e) {
        const float partner = __shfl_xor_sync(0xffffffffu, x[e], 4);
        if (ln < 8) {
            const int i = (8 * ln + e) & 31;
            const float ang = __fmul_rn((float)rope_pos, inv_freq[i]);
            const float c = cosf(ang), s = sinf(ang);
            const float sw = ln < 4 ? -partner : partner;
            x[e] = __fadd_rn(__fmul_rn(x[e], c), __fmul_rn(sw, s));
        }
    }
}

__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
    return make_uint4(pack_bf2(f[0], f[1]), pack_bf2(f[2], f[3]), pack_bf2(f[4], f[5]),
                      pack_bf2(f[6], f[7]));
}

__device__ __forceinline__ size_t kv_offset(const int* __restrict__ table, int pos, int kvh) {
    const int page = table[pos / kKvPage];
    return (size_t)page * kPageElems + ((size_t)kvh * kKvPage + (pos % kKvPage)) * kHeadDim;
}

// Append k (normed, roped, bf16) and raw v of one row to the cache.  Executed by two warps.
__device__ __forceinline__ void append_kv(const AttnParams& p, const uint16_t* __restrict__ pr,
                                          const int* __restrict__ table, int kvh, int slot,
                                          int rope_pos, int which, int ln) {
    if (which == 0) {
        float x[8];
        unpack8(*reinterpret_cast<const uint4*>(pr + kOffK + kvh * kHeadDim + 8 * ln), x);
        head_norm_rope(x, p.k_norm, ln, rope_pos, p.inv_freq);
        *reinterpret_cast<uint4*>(p.kpool + kv_offset(table, slot, kvh) + 8 * ln) = pack8(x);
    } else {
        *reinterpret_cast<uint4*>(p.vpool + kv_offset(table, slot, kvh) + 8 * ln) =
            *reinterpret_cast<const uint4*>(pr + kOffV + kvh * kHeadDim + 8 * ln);
    }
}

// grid (rows, 2 kv heads), 64 threads: used when a body carries T > 1 rows per lane, so that every
// row's K/V is in the cache before any row's scores are taken.
__global__ void __launch_bounds__(64) attn_append_kernel(AttnParams p) {
    const int row = blockIdx.x, kvh = blockIdx.y;
    const int lane_id = row / p.T, t = row % p.T;
    const int slot = p.slot[lane_id] + t;
    if (slot >= p.pages_per_lane * kKvPage) return;
    const int* table = p.page_table + (size_t)lane_id * p.table_lane_stride;
    append_kv(p, p.proj + (size_t)row * kAttnProjN, table, kvh, slot, p.rope_pos[lane_id] + t,
              threadIdx.x >> 5, threadIdx.x & 31);
}

template <bool FUSED_APPEND>
__global__ void __launch_bounds__(256, 2) attn_decode_kernel(AttnParams p, int ctx_pad) {
    extern __shared__ __align__(16) float smem[];
    float* q_s = smem;                       // [4][256]
    float* part = smem + 4 * kHeadDim;       // [8][4][256]
    float* sc = part + 8 * 4 * kHeadDim;     // [4][ctx_pad]

    const int row = blockIdx.x, kvh = blockIdx.y;
    const int tid = threadIdx.x, warp = tid >> 5, ln = tid & 31;
    const int lane_id = row / p.T, t = row % p.T;
    const int cap = p.pages_per_lane * kKvPage;
    int slot = p.slot[lane_id] + t;
    const int rope_pos = p.rope_pos[lane_id] + t;
    const bool in_cap = slot < cap && slot < ctx_pad;
    if (!in_cap) slot = (cap < ctx_pad ? cap : ctx_pad) - 1;   // never index past the cache; host checks capacity
    const int n_ctx = slot + 1;
    const int* table = p.page_table + (size_t)lane_id * p.table_lane_stride;
    const uint16_t* pr = p.proj + (size_t)row * kAttnProjN;

    // ---- q heads: norm + rope -> shared; k/v of this row -> cache ------------------------------
    if (warp < 4) {
        const int head = kvh * 4 + warp;
        float x[8];
        unpack8(*reinterpret_cast<const uint4*>(pr + head * 2 * kHeadDim + 8 * ln), x);
        head_norm_rope(x, p.q_norm, ln, rope_pos, p.inv_freq);
#pragma unroll
        for (int e = 0; e < 8; ++e) q_s[warp * kHeadDim + 8 * ln + e] = x[e];
    } else if (FUSED_APPEND && warp < 6 && in_cap) {
        append_kv(p, pr, table, kvh, slot, rope_pos, warp - 4, ln);
    }
    __syncthreads();

    // ---- scores: s[h][pos] = (q_h . K[pos]) / 16 ----------------------------------------------
    {
        float qr[4][8];
#pragma unroll
        for (int hh = 0; hh < 4; ++hh)
#pragma unroll
            for (int e = 0; e < 8; ++e) qr[hh][e] = q_s[hh * kHeadDim + 8 * ln + e];
        for (int p0 = warp * 4; p0 < n_ctx; p0 += 32) {
            const size_t base = kv_offset(table, p0, kvh) + 8 * ln;   // 4 positions share a page
            uint4 kv[4];
#pragma unroll
            for (int u = 0; u < 4; ++u)
                kv[u] = (p0 + u < n_ctx) ? *reinterpret_cast<const uint4*>(p.kpool + base + u * kHeadDim)
                                         : make_uint4(0, 0, 0, 0);
            float d[4][4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                float kf[8];
                unpack8(kv[u], kf);
#pragma unroll
                for (int hh = 0; hh < 4; ++hh) {
                    float a = 0.f;
#pragma unroll
                    for (int e = 0; e < 8; ++e) a += qr[hh][e] * kf[e];
                    d[u][hh] = a;
                }
            }
#pragma unroll
            for (int u = 0; u < 4; ++u)
#pragma unroll
                for (int hh = 0; hh < 4; ++hh) d[u][hh] = warp_sum(d[u][hh]);
            if (ln < 16) {
                const int u = ln >> 2, hh = ln & 3;
                float v = 0.f;
#pragma unroll
                for (int uu = 0; uu < 4; ++uu)
#pragma unroll
                    for (int h2 = 0; h2 < 4; ++h2)
                        if (uu == u && h2 == hh) v = d[uu][h2];
                if (p0 + u < n_ctx) sc[hh * ctx_pad + p0 + u] = v * 0.0625f;
            }
        }
    }
    __syncthreads();

    // ---- softmax per head (f32), weights rounded to bf16 ---------------------------------------
    if (warp < 4) {
        float* s = sc + warp * ctx_pad;
        float m = -INFINITY;
        for (int i = ln; i < n_ctx; i += 32) m = fmaxf(m, s[i]);
        m = warp_max(m);
        float l = 0.f;
        for (int i = ln; i < n_ctx; i += 32) {
            const float e = expf(s[i] - m);
            s[i] = e;
            l += e;
        }
        l = warp_sum(l);
        for (int i = ln; i < n_ctx; i += 32) s[i] = bfround(__fdiv_rn(s[i], l));
    }
    __syncthreads();

    // ---- P.V: each warp takes positions p0..p0+3 (stride 32), lane holds 8 dims ----------------
    {
        float acc[4][8];
#pragma unroll
        for (int hh = 0; hh < 4; ++hh)
#pragma unroll
            for (int e = 0; e < 8; ++e) acc[hh][e] = 0.f;
        for (int p0 = warp * 4; p0 < n_ctx; p0 += 32) {
            const size_t base = kv_offset(table, p0, kvh) + 8 * ln;
            uint4 vv[4];
#pragma unroll
            for (int u = 0; u < 4; ++u)
                vv[u] = (p0 + u < n_ctx) ? *reinterpret_cast<const uint4*>(p.vpool + base + u * kHeadDim)
                                         : make_uint4(0, 0, 0, 0);
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                if (p0 + u >= n_ctx) break;
                float vf[8];
                unpack8(vv[u], vf);
#pragma unroll
                for (int hh = 0; hh < 4; ++hh) {
                    const float wgt = sc[hh * ctx_pad + p0 + u];
#pragma unroll
                    for (int e = 0; e < 8; ++e) acc[hh][e] += wgt * vf[e];
                }
            }
        }
#pragma unroll
        for (int hh = 0; hh < 4; ++hh) {
            float4* dst = reinterpret_cast<float4*>(part + ((warp * 4 + hh) * kHeadDim) + 8 * ln);
            dst[0] = make_float4(acc[hh][0], acc[hh][1], acc[hh][2], acc[hh][3]);
            dst[1] = make_float4(acc[hh][4], acc[hh][5], acc[hh][6], acc[hh][7]);
        }
    }
    __syncthreads();

    // ---- combine warps, round, apply the bf16 sigmoid gate --------------------------------------
    for (int idx = tid; idx < 4 * kHeadDim; idx += 256) {
        const int hh = idx >> 8, dd = idx & 255;
        float a = 0.f;
#pragma unroll
        for (int w = 0; w < 8; ++w) a += part[(w * 4 + hh) * kHeadDim + dd];
        a = bfround(a);
        const int head = kvh * 4 + hh;
        const float gate = bf2f(pr[head * 2 * kHeadDim + kHeadDim + dd]);
        const float sg = bfround(sigmoid_acc(gate));
        p.out[(size_t)row * (kQHeads * kHeadDim) + head * kHeadDim + dd] = f2bf(a * sg);
    }
}

static size_t attn_smem_bytes(int ctx_pad) {
    return (size_t)(4 * kHeadDim + 8 * 4 * kHeadDim + 4 * ctx_pad) * sizeof(float);
}

cudaError_t attn_init() {
    const int max_bytes = (int)attn_smem_bytes(kAttnMaxCtx);
    cudaError_t e = cudaFuncSetAttribute(attn_decode_kernel<true>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, max_bytes);
    if (e != cudaSuccess) return e;
    return cudaFuncSetAttribute(attn_decode_kernel<false>,
                                cudaFuncAttributeMaxDynamicSharedMemorySize, max_bytes);
}

cudaError_t launch_attn(const AttnParams& p, cudaStream_t st) {
    if (p.lanes <= 0 || p.T <= 0 || p.max_ctx <= 0 || p.max_ctx > kAttnMaxCtx) return cudaErrorInvalidValue;
    const int ctx_pad = (p.max_ctx + 31) & ~31;
    const int rows = p.lanes * p.T;
    const dim3 grid(rows, kKvHeads);
    const size_t smem = attn_smem_bytes(ctx_pad);
    if (p.T == 1) {
        attn_decode_kernel<true><<<grid, 256, smem, st>>>(p, ctx_pad);
    } else {
        attn_append_kernel<<<grid, 64, 0, st>>>(p);
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) return e;
        attn_decode_kernel<false><<<grid, 256, smem, st>>>(p, ctx_pad);
    }
    return cudaGetLastError();
}

}  // namespace q35
