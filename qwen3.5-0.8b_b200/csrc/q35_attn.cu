// Gated GQA decode attention over a paged KV cache: per-head RMSNorm of q and k, partial RoPE on
// dims 0..63 (pairs i, i+32), KV append, f32 scores and softmax, bf16 softmax weights, P.V, and
// the sigmoid output gate, in one kernel.
//
// One CTA per (row, kv head): the 4 query heads that share a KV head are processed together so
// every cached K and V row is read from HBM once per row.  A warp reads a whole 512-byte K (or V)
// row with 16-byte loads; the cache is addressed through a per-lane page table
// (page = 64 positions x 2 kv heads x 256 dims).
//
// Two forms.  Context capacities up to 3072 positions: attn_tma_kernel streams whole K and V pages (32 KiB per
// kv head) through a two-deep shared-memory ring with TMA (128-byte swizzle), takes the scores and
// P.V on the tensor cores (m16n8k16; q is split into bf16 hi + lo parts so the f32 rotated query
// loses nothing, the softmax weights are bf16 by contract), and keeps two CTAs per SM (up to 1024
// positions) so four pages are in flight per SM.  Longer contexts: attn_decode_kernel (plain loads, CUDA-core dots).
//
// Replaces attn_decode_layer / mtp_attn_row (engine/kernels.h:730-906,
// engine/kernels_attn.cpp:995-1068); arithmetic follows speccheck/specimpl.py:320-397 as executed,
// except that cached keys are bf16 (the engine's cache dtype, engine/state.h:90).
#include <cuda.h>

#include <cstdlib>

#include "q35_common.cuh"
#include "q35_async.cuh"

namespace q35 {

constexpr int kAttnMaxCtx = 8192;
// Context capacities up to here take the TMA + tensor-core forms: their scores and weights of the whole
// row live in shared memory (40 bytes per position beside the 64 KiB page ring), so up to 1,024
// positions two CTAs share an SM and beyond that one CTA has it alone.
constexpr int kAttnTmaMaxCtx = 3072;
constexpr int kOffK = 4096, kOffV = 4608;

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
    pdl_wait();
    pdl_trigger();          // the attention kernel behind this one reads the cache only after its own wait
    const int row = blockIdx.x, kvh = blockIdx.y;
    const int lane_id = row / p.T, t = row % p.T;
    const int slot = p.slot[lane_id] + t;
    if (slot < 0 || slot >= p.pages_per_lane * kKvPage) return;
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

    pdl_wait();
    const int row = blockIdx.x, kvh = blockIdx.y;
    const int tid = threadIdx.x, warp = tid >> 5, ln = tid & 31;
    const int lane_id = row / p.T, t = row % p.T;
    const int cap = p.pages_per_lane * kKvPage;
    int slot = p.slot[lane_id] + t;
    const int rope_pos = p.rope_pos[lane_id] + t;
    const bool in_cap = slot >= 0 && slot < cap && slot < ctx_pad;   // a negative slot (a state driven out of order) is never indexed
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


// ------------------------------------------------------------------------------------------------
// TMA + tensor-core form (context capacities <= kAttnTmaMaxCtx)
// ------------------------------------------------------------------------------------------------
namespace {

constexpr int kTileBytes = kKvPage * kHeadDim * 2;        // one kv head's slice of a page: 32 KiB
constexpr int kRing = 2;
constexpr int kTmaThreads = 288;                          // 8 consumer warps + 1 producer warp

__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// byte offset of (row, 16-byte chunk of a 256-wide bf16 row) inside a TMA-swizzled page tile:
// four column blocks of [64 rows][128 B], chunk index XOR (row & 7) within a block
__device__ __forceinline__ uint32_t tile_off(int row, int chunk32) {
    const int cb = chunk32 >> 3, c = chunk32 & 7;
    return (uint32_t)(cb * 8192 + row * 128 + ((c ^ (row & 7)) << 4));
}

template <bool FUSED_APPEND>
__global__ void __launch_bounds__(kTmaThreads, 2)
attn_tma_kernel(AttnParams p, int ctx_pad, const __grid_constant__ CUtensorMap kmap,
                const __grid_constant__ CUtensorMap vmap) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) unsigned long long bars[2 * kRing];
    if (threadIdx.x == 0) { prefetch_tensormap(&kmap); prefetch_tensormap(&vmap); }
    pdl_wait();
    pdl_trigger();          // the output projection behind this kernel may start fetching its weights
    if (p.status != nullptr && *p.status != 0) return;

    const uint32_t ring = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* base_ptr = smem_raw + (ring - smem_u32(smem_raw));
    float* q_s = reinterpret_cast<float*>(base_ptr + kRing * kTileBytes);      // [4][256]
    float* sc2 = q_s + 4 * kHeadDim;                                           // [2][4][ctx_pad]
    uint16_t* w_s = reinterpret_cast<uint16_t*>(sc2 + 8 * ctx_pad);            // [4][ctx_pad] bf16
    const uint32_t full0 = smem_u32(&bars[0]), empty0 = smem_u32(&bars[kRing]);

    const int row = blockIdx.x, kvh = blockIdx.y;
    const int tid = threadIdx.x, warp = tid >> 5, ln = tid & 31;
    const int g = ln >> 2, t = ln & 3;
    const int lane_id = row / p.T, tt = row % p.T;
    const int cap = p.pages_per_lane * kKvPage;
    int slot = p.slot[lane_id] + tt;
    const int rope_pos = p.rope_pos[lane_id] + tt;
    const bool in_cap = slot >= 0 && slot < cap && slot < ctx_pad;   // a negative slot (a state driven out of order) is never indexed
    if (!in_cap) slot = (cap < ctx_pad ? cap : ctx_pad) - 1;
    const int n_ctx = slot + 1;
    const int P = (n_ctx + kKvPage - 1) / kKvPage;          // pages (tiles) per pass
    const int* table = p.page_table + (size_t)lane_id * p.table_lane_stride;
    const uint16_t* pr = p.proj + (size_t)row * kAttnProjN;

    if (tid == 0) {
        for (int b = 0; b < kRing; ++b) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;\n" ::"r"(full0 + 8 * b) : "memory");
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 8;\n" ::"r"(empty0 + 8 * b) : "memory");
        }
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    __syncthreads();

    // tile i of 2P: K pages 0..P-1, then V pages 0..P-1
    auto issue = [&](int i) -> bool {
        const int b = i % kRing;
        const uint32_t ph = (i / kRing) & 1;
        if (!mbar_wait(empty0 + 8 * b, ph ^ 1)) return false;
        const int page = table[i < P ? i : i - P];
        const CUtensorMap* map = i < P ? &kmap : &vmap;
        const uint32_t dst = ring + b * kTileBytes;
        const int r0 = page * (kKvHeads * kKvPage) + kvh * kKvPage;
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(full0 + 8 * b), "r"(kTileBytes) : "memory");
#pragma unroll
        for (int cb = 0; cb < 4; ++cb)
            asm volatile(
                "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n"
                ::"r"(dst + cb * 8192), "l"(reinterpret_cast<uint64_t>(map)), "r"(full0 + 8 * b), "r"(cb * 64), "r"(r0) : "memory");
        return true;
    };

    // ---- prologue: producer starts the pages that do not hold the new row; q / k / v prep -------
    int issued = 0;
    bool prod_ok = true;
    if (warp == 8) {
        if (ln == 0) {
            const int safe = FUSED_APPEND ? (P - 1) : 2 * P;
            while (issued < kRing && issued < safe && prod_ok) { prod_ok = issue(issued); ++issued; }
        }
    } else if (warp < 4) {
        const int head = kvh * 4 + warp;
        float x[8];
        unpack8(*reinterpret_cast<const uint4*>(pr + head * 2 * kHeadDim + 8 * ln), x);
        head_norm_rope(x, p.q_norm, ln, rope_pos, p.inv_freq);
#pragma unroll
        for (int e = 0; e < 8; ++e) q_s[warp * kHeadDim + 8 * ln + e] = x[e];
    } else if (FUSED_APPEND && warp < 6 && in_cap) {
        append_kv(p, pr, table, kvh, slot, rope_pos, warp - 4, ln);
        __threadfence();
        asm volatile("fence.proxy.async;\n" ::: "memory");       // the new row must be visible to the TMA reads below
    }
    __syncthreads();

    if (warp == 8) {
        if (ln == 0) {
            while (issued < 2 * P && prod_ok) { prod_ok = issue(issued); ++issued; }
            if (!prod_ok && p.status != nullptr) atomicExch(p.status, 5);
        }
        return;
    }

    // ---- pass 1: scores.  warp = (16-position m-tile, 128-dim half) of every K page ---------------
    bool ok = true;
    {
        const int mt = warp & 3, kh = warp >> 2;
        uint32_t bhi[8][2], blo[8][2];
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                float v0 = 0.f, v1 = 0.f;
                if (g < 4) {
                    const int d = kh * 128 + ks * 16 + half * 8 + 2 * t;
                    v0 = q_s[g * kHeadDim + d];
                    v1 = q_s[g * kHeadDim + d + 1];
                }
                const float h0 = bfround(v0), h1 = bfround(v1);
                bhi[ks][half] = pack_bf2(h0, h1);
                blo[ks][half] = pack_bf2(v0 - h0, v1 - h1);
            }
        for (int i = 0; i < P; ++i) {
            const int b = i % kRing;
            if (ok) ok = mbar_wait(full0 + 8 * b, (i / kRing) & 1);
            const uint32_t tile = ring + b * kTileBytes;
            float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int ks = 0; ks < 8; ++ks) {
                uint32_t a[4];
                const int r = mt * 16 + (ln & 15);
                ldsm_x4(a, tile + tile_off(r, kh * 16 + ks * 2 + (ln >> 4)));
                mma_bf16(acc, a[0], a[1], a[2], a[3], bhi[ks][0], bhi[ks][1]);
                mma_bf16(acc, a[0], a[1], a[2], a[3], blo[ks][0], blo[ks][1]);
            }
            if (t < 2) {
                const int pos = i * kKvPage + mt * 16 + g;
                float* s0 = sc2 + (kh * 4 + 2 * t) * ctx_pad;
                if (pos < ctx_pad) { s0[pos] = acc[0] * 0.0625f; s0[ctx_pad + pos] = acc[1] * 0.0625f; }
                if (pos + 8 < ctx_pad) { s0[pos + 8] = acc[2] * 0.0625f; s0[ctx_pad + pos + 8] = acc[3] * 0.0625f; }
            }
            __syncwarp();
            if (ln == 0) mbar_arrive(empty0 + 8 * b);
        }
    }
    asm volatile("bar.sync 1, 256;\n" ::: "memory");

    // ---- softmax per head (f32), weights rounded to bf16, zero past the context ------------------
    if (warp < 4) {
        const float* sa = sc2 + warp * ctx_pad;
        const float* sb = sc2 + (4 + warp) * ctx_pad;
        float m = -INFINITY;
        for (int i = ln; i < n_ctx; i += 32) m = fmaxf(m, sa[i] + sb[i]);
        m = warp_max(m);
        float l = 0.f;
        for (int i = ln; i < n_ctx; i += 32) l += expf(sa[i] + sb[i] - m);
        l = warp_sum(l);
        uint16_t* w = w_s + warp * ctx_pad;
        for (int i = ln; i < P * kKvPage && i < ctx_pad; i += 32)
            w[i] = i < n_ctx ? f2bf(__fdiv_rn(expf(sa[i] + sb[i] - m), l)) : (uint16_t)0;
    }
    asm volatile("bar.sync 1, 256;\n" ::: "memory");

    // ---- pass 2: P.V.  warp = 32 output dims; heads ride in rows 0..3 of the m16 tile -------------
    float acc[4][4];
#pragma unroll
    for (int nt = 0; nt < 4; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[nt][e] = 0.f;
    for (int i = 0; i < P; ++i) {
        const int ti = P + i, b = ti % kRing;
        if (ok) ok = mbar_wait(full0 + 8 * b, (ti / kRing) & 1);
        const uint32_t tile = ring + b * kTileBytes;
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
            const int p0 = i * kKvPage + ks * 16;
            uint32_t a0 = 0, a2 = 0;
            if (g < 4 && p0 + 16 <= ctx_pad) {
                a0 = *reinterpret_cast<const uint32_t*>(w_s + g * ctx_pad + p0 + 2 * t);
                a2 = *reinterpret_cast<const uint32_t*>(w_s + g * ctx_pad + p0 + 8 + 2 * t);
            }
#pragma unroll
            for (int np = 0; np < 2; ++np) {
                uint32_t r[4];
                const int pos = ks * 16 + (ln & 7) + ((ln >> 3) & 1) * 8;
                ldsm_x4_trans(r, tile + tile_off(pos, warp * 4 + np * 2 + (ln >> 4)));
                mma_bf16(acc[2 * np], a0, 0u, a2, 0u, r[0], r[1]);
                mma_bf16(acc[2 * np + 1], a0, 0u, a2, 0u, r[2], r[3]);
            }
        }
        __syncwarp();
        if (ln == 0) mbar_arrive(empty0 + 8 * b);
    }
    if (!ok) {
        if (ln == 0 && p.status != nullptr) atomicExch(p.status, 6);
        return;
    }

    // ---- epilogue: round, apply the bf16 sigmoid gate ---------------------------------------------
    if (g < 4) {
        const int head = kvh * 4 + g;
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
            const int dd = warp * 32 + nt * 8 + 2 * t;
            const uint32_t gw = *reinterpret_cast<const uint32_t*>(pr + head * 2 * kHeadDim + kHeadDim + dd);
            const float o0 = bfround(acc[nt][0]) * bfround(sigmoid_acc(lo_bf(gw)));
            const float o1 = bfround(acc[nt][1]) * bfround(sigmoid_acc(hi_bf(gw)));
            *reinterpret_cast<uint32_t*>(p.out + (size_t)row * (kQHeads * kHeadDim) + head * kHeadDim + dd) = pack_bf2(o0, o1);
        }
    }
}

// ------------------------------------------------------------------------------------------------
// Cluster form for bodies of few rows: a thread-block cluster of CS CTAs shares one (row, kv head).
// CTA `rank` takes the pages i = rank, rank + CS, ... of the lane's context, so a 560-position
// context is read by 8 CTAs at once instead of one CTA walking 18 tiles.  The rounding points of the
// single-CTA form are kept: scores f32; ONE softmax over the whole row - every CTA publishes its
// local (max, sum of exp), all combine them in rank order to the row's max M and sum L, and the
// weights bf16(exp(s - M) / L) are final before P.V; the f32 partial outputs are summed through
// distributed shared memory in rank order (rank r sums and stores its 256 / CS slice of the dims).
// Every CTA runs the same three cluster barriers whatever happens (a dead status word, an expired
// wait): nothing in a cluster ever waits for a CTA that left early.
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ void cluster_sync_all() {
    __syncwarp();                      // the aligned barrier needs the whole warp at this instruction
    asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}
__device__ __forceinline__ uint32_t peer_addr(const void* p, uint32_t rank) {
    uint32_t ra;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(ra) : "r"(smem_u32(p)), "r"(rank));
    return ra;
}
__device__ __forceinline__ float peer_ld_f32(uint32_t addr) {
    float v;
    asm volatile("ld.shared::cluster.f32 %0, [%1];\n" : "=f"(v) : "r"(addr) : "memory");
    return v;
}
__device__ __forceinline__ float2 peer_ld_f32x2(uint32_t addr) {
    float2 v;
    asm volatile("ld.shared::cluster.v2.f32 {%0, %1}, [%2];\n" : "=f"(v.x), "=f"(v.y) : "r"(addr) : "memory");
    return v;
}

template <bool FUSED_APPEND>
__global__ void __launch_bounds__(kTmaThreads, 2)
attn_cluster_kernel(AttnParams p, int ctx_pad, int lpad, int cs, const __grid_constant__ CUtensorMap kmap,
                    const __grid_constant__ CUtensorMap vmap) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) unsigned long long bars[2 * kRing];
    if (threadIdx.x == 0) { prefetch_tensormap(&kmap); prefetch_tensormap(&vmap); }
    __shared__ float ml_s[8];                              // local max [4 heads] | local sum of exp [4]
    __shared__ __align__(16) float o_part[4 * kHeadDim];   // this CTA's f32 partial of P.V
    pdl_wait();
    pdl_trigger();          // the output projection behind this kernel may start fetching its weights
    const bool dead = p.status != nullptr && *p.status != 0;

    const uint32_t ring = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* base_ptr = smem_raw + (ring - smem_u32(smem_raw));
    float* q_s = reinterpret_cast<float*>(base_ptr + kRing * kTileBytes);      // [4][256]
    // scores and weights of THIS CTA's pages only, page j of the CTA at [j * 64, j * 64 + 64): lpad = 64 x the
    // most pages a CTA of the cluster can own, so the footprint falls with the cluster size
    float* sc2 = q_s + 4 * kHeadDim;                                           // [2][4][lpad]
    uint16_t* w_s = reinterpret_cast<uint16_t*>(sc2 + 8 * lpad);               // [4][lpad] bf16
    const uint32_t full0 = smem_u32(&bars[0]), empty0 = smem_u32(&bars[kRing]);

    const int row = blockIdx.x, kvh = blockIdx.y, rank = blockIdx.z;
    const int tid = threadIdx.x, warp = tid >> 5, ln = tid & 31;
    const int g = ln >> 2, t = ln & 3;
    const int lane_id = row / p.T, tt = row % p.T;
    const int cap = p.pages_per_lane * kKvPage;
    int slot = p.slot[lane_id] + tt;
    const int rope_pos = p.rope_pos[lane_id] + tt;
    const bool in_cap = slot >= 0 && slot < cap && slot < ctx_pad;   // a negative slot (a state driven out of order) is never indexed
    if (!in_cap) slot = (cap < ctx_pad ? cap : ctx_pad) - 1;
    const int n_ctx = slot + 1;
    const int P = (n_ctx + kKvPage - 1) / kKvPage;                       // pages of the whole context
    const int myP = dead ? 0 : (P > rank ? (P - rank + cs - 1) / cs : 0); // pages this CTA reads: rank + j * cs
    const bool owner = ((P - 1) % cs) == rank;                           // this CTA's last page holds the new row
    const int* table = p.page_table + (size_t)lane_id * p.table_lane_stride;
    const uint16_t* pr = p.proj + (size_t)row * kAttnProjN;

    if (tid == 0) {
        for (int b = 0; b < kRing; ++b) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;\n" ::"r"(full0 + 8 * b) : "memory");
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 8;\n" ::"r"(empty0 + 8 * b) : "memory");
        }
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    __syncthreads();

    // tile j of 2 * myP: this CTA's K pages, then its V pages
    auto issue = [&](int j) -> bool {
        const int b = j % kRing;
        const uint32_t ph = (j / kRing) & 1;
        if (!mbar_wait(empty0 + 8 * b, ph ^ 1)) return false;
        const int page = table[rank + (j < myP ? j : j - myP) * cs];
        const CUtensorMap* map = j < myP ? &kmap : &vmap;
        const uint32_t dst = ring + b * kTileBytes;
        const int r0 = page * (kKvHeads * kKvPage) + kvh * kKvPage;
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(full0 + 8 * b), "r"(kTileBytes) : "memory");
#pragma unroll
        for (int cb = 0; cb < 4; ++cb)
            asm volatile(
                "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n"
                ::"r"(dst + cb * 8192), "l"(reinterpret_cast<uint64_t>(map)), "r"(full0 + 8 * b), "r"(cb * 64), "r"(r0) : "memory");
        return true;
    };

    // ---- prologue: the producer starts the pages that do not hold the new row; q / k / v prep -------
    int issued = 0;
    bool prod_ok = true;
    if (warp == 8) {
        if (ln == 0) {
            const int safe = (FUSED_APPEND && owner) ? (myP - 1) : 2 * myP;
            while (issued < kRing && issued < safe && prod_ok) { prod_ok = issue(issued); ++issued; }
        }
    } else if (warp < 4) {
        const int head = kvh * 4 + warp;
        float x[8];
        unpack8(*reinterpret_cast<const uint4*>(pr + head * 2 * kHeadDim + 8 * ln), x);
        head_norm_rope(x, p.q_norm, ln, rope_pos, p.inv_freq);
#pragma unroll
        for (int e = 0; e < 8; ++e) q_s[warp * kHeadDim + 8 * ln + e] = x[e];
    } else if (FUSED_APPEND && warp < 6 && in_cap && owner && !dead) {
        append_kv(p, pr, table, kvh, slot, rope_pos, warp - 4, ln);
        __threadfence();
        asm volatile("fence.proxy.async;\n" ::: "memory");       // the new row must be visible to the TMA reads below
    }
    __syncthreads();

    bool ok = true;
    float acc[4][4];
#pragma unroll
    for (int nt = 0; nt < 4; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[nt][e] = 0.f;

    if (warp == 8) {
        if (ln == 0) {
            // Only tiles whose ring slot pass 1 frees may be issued before the cluster barrier below:
            // a later tile waits for a release of pass 2, which starts after that barrier.
            const int before = (myP + kRing) < 2 * myP ? (myP + kRing) : 2 * myP;
            while (issued < before && prod_ok) { prod_ok = issue(issued); ++issued; }
        }
    } else {
        // ---- pass 1: scores of this CTA's pages.  warp = (16-position m-tile, 128-dim half) --------
        const int mt = warp & 3, kh = warp >> 2;
        uint32_t bhi[8][2], blo[8][2];
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                float v0 = 0.f, v1 = 0.f;
                if (g < 4) {
                    const int d = kh * 128 + ks * 16 + half * 8 + 2 * t;
                    v0 = q_s[g * kHeadDim + d];
                    v1 = q_s[g * kHeadDim + d + 1];
                }
                const float h0 = bfround(v0), h1 = bfround(v1);
                bhi[ks][half] = pack_bf2(h0, h1);
                blo[ks][half] = pack_bf2(v0 - h0, v1 - h1);
            }
        for (int j = 0; j < myP; ++j) {
            const int b = j % kRing;
            if (ok) ok = mbar_wait(full0 + 8 * b, (j / kRing) & 1);
            const uint32_t tile = ring + b * kTileBytes;
            float sacc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int ks = 0; ks < 8; ++ks) {
                uint32_t a[4];
                const int r = mt * 16 + (ln & 15);
                ldsm_x4(a, tile + tile_off(r, kh * 16 + ks * 2 + (ln >> 4)));
                mma_bf16(sacc, a[0], a[1], a[2], a[3], bhi[ks][0], bhi[ks][1]);
                mma_bf16(sacc, a[0], a[1], a[2], a[3], blo[ks][0], blo[ks][1]);
            }
            if (t < 2) {
                const int pos = j * kKvPage + mt * 16 + g;               // local: j < myP <= lpad / 64
                float* s0 = sc2 + (kh * 4 + 2 * t) * lpad;
                s0[pos] = sacc[0] * 0.0625f; s0[lpad + pos] = sacc[1] * 0.0625f;
                s0[pos + 8] = sacc[2] * 0.0625f; s0[lpad + pos + 8] = sacc[3] * 0.0625f;
            }
            __syncwarp();
            if (ln == 0) mbar_arrive(empty0 + 8 * b);
        }
        asm volatile("bar.sync 1, 256;\n" ::: "memory");
        // ---- local max and sum of exp per head over this CTA's positions ----------------------------
        if (warp < 4) {
            const float* sa = sc2 + warp * lpad;
            const float* sb = sc2 + (4 + warp) * lpad;
            float m = -INFINITY;
            for (int j = 0; j < myP; ++j) {
                const int left = n_ctx - (rank + j * cs) * kKvPage;     // positions of this page inside the context
                for (int o = ln; o < kKvPage && o < left; o += 32) m = fmaxf(m, sa[j * kKvPage + o] + sb[j * kKvPage + o]);
            }
            m = warp_max(m);
            float l = 0.f;
            for (int j = 0; j < myP; ++j) {
                const int left = n_ctx - (rank + j * cs) * kKvPage;
                for (int o = ln; o < kKvPage && o < left; o += 32) l += expf(sa[j * kKvPage + o] + sb[j * kKvPage + o] - m);
            }
            l = warp_sum(l);
            if (ln == 0) { ml_s[warp] = m; ml_s[4 + warp] = l; }
        }
    }
    cluster_sync_all();                                    // (1) every CTA's (max, sum) is published

    if (warp == 8 && ln == 0) {
        while (issued < 2 * myP && prod_ok) { prod_ok = issue(issued); ++issued; }
        if (!prod_ok && p.status != nullptr) atomicExch(p.status, 5);
    }
    if (warp < 4) {
        // the row's max and sum, combined in rank order: identical in every CTA of the cluster
        float M = -INFINITY;
        for (int r = 0; r < cs; ++r) M = fmaxf(M, peer_ld_f32(peer_addr(&ml_s[warp], r)));
        float L = 0.f;
        for (int r = 0; r < cs; ++r) {
            const float mr = peer_ld_f32(peer_addr(&ml_s[warp], r)), lr = peer_ld_f32(peer_addr(&ml_s[4 + warp], r));
            if (lr > 0.f) L += lr * expf(mr - M);
        }
        const float* sa = sc2 + warp * lpad;
        const float* sb = sc2 + (4 + warp) * lpad;
        uint16_t* w = w_s + warp * lpad;
        for (int j = 0; j < myP; ++j) {
            const int left = n_ctx - (rank + j * cs) * kKvPage;
            for (int o = ln; o < kKvPage; o += 32) {
                const int i = j * kKvPage + o;
                w[i] = o < left ? f2bf(__fdiv_rn(expf(sa[i] + sb[i] - M), L)) : (uint16_t)0;
            }
        }
    }
    if (warp < 8) {
        asm volatile("bar.sync 1, 256;\n" ::: "memory");
        // ---- pass 2: P.V over this CTA's pages.  warp = 32 output dims; heads ride in rows 0..3 -----
        for (int j = 0; j < myP; ++j) {
            const int tj = myP + j, b = tj % kRing;
            if (ok) ok = mbar_wait(full0 + 8 * b, (tj / kRing) & 1);
            const uint32_t tile = ring + b * kTileBytes;
#pragma unroll
            for (int ks = 0; ks < 4; ++ks) {
                const int p0 = j * kKvPage + ks * 16;
                uint32_t a0 = 0, a2 = 0;
                if (g < 4) {
                    a0 = *reinterpret_cast<const uint32_t*>(w_s + g * lpad + p0 + 2 * t);
                    a2 = *reinterpret_cast<const uint32_t*>(w_s + g * lpad + p0 + 8 + 2 * t);
                }
#pragma unroll
                for (int np = 0; np < 2; ++np) {
                    uint32_t r[4];
                    const int pos = ks * 16 + (ln & 7) + ((ln >> 3) & 1) * 8;
                    ldsm_x4_trans(r, tile + tile_off(pos, warp * 4 + np * 2 + (ln >> 4)));
                    mma_bf16(acc[2 * np], a0, 0u, a2, 0u, r[0], r[1]);
                    mma_bf16(acc[2 * np + 1], a0, 0u, a2, 0u, r[2], r[3]);
                }
            }
            __syncwarp();
            if (ln == 0) mbar_arrive(empty0 + 8 * b);
        }
        if (!ok && ln == 0 && p.status != nullptr) atomicExch(p.status, 6);
        if (g < 4) {
#pragma unroll
            for (int nt = 0; nt < 4; ++nt) {
                const int dd = warp * 32 + nt * 8 + 2 * t;
                *reinterpret_cast<float2*>(&o_part[g * kHeadDim + dd]) = make_float2(acc[nt][0], acc[nt][1]);
            }
        }
    }
    cluster_sync_all();                                    // (2) every CTA's partial output is published

    // ---- rank r sums dims [r * DS, (r + 1) * DS) of the four heads in rank order, gates, stores -----
    {
        const int DS = kHeadDim / cs;
        const bool alive = !dead && (p.status == nullptr || *p.status == 0);
        if (tid < 2 * DS && alive) {
            const int hh = tid / (DS / 2), dd = rank * DS + 2 * (tid % (DS / 2));
            float2 sum = make_float2(0.f, 0.f);
            for (int r = 0; r < cs; ++r) {
                const float2 v = peer_ld_f32x2(peer_addr(&o_part[hh * kHeadDim + dd], r));
                sum.x += v.x; sum.y += v.y;
            }
            const int head = kvh * 4 + hh;
            const uint32_t gw = *reinterpret_cast<const uint32_t*>(pr + head * 2 * kHeadDim + kHeadDim + dd);
            const float o0 = bfround(sum.x) * bfround(sigmoid_acc(lo_bf(gw)));
            const float o1 = bfround(sum.y) * bfround(sigmoid_acc(hi_bf(gw)));
            *reinterpret_cast<uint32_t*>(p.out + (size_t)row * (kQHeads * kHeadDim) + head * kHeadDim + dd) = pack_bf2(o0, o1);
        }
    }
    cluster_sync_all();                                    // (3) no CTA leaves while a peer may still read it
}

// ------------------------------------------------------------------------------------------------
// Prompt bodies: causal attention of a block of 16 consecutive rows of one lane.
// The row-by-row forms above read a lane's whole context once per row; a prompt body carries up to
// 64 rows per lane, so here one CTA takes 16 rows x the 4 q heads of a kv head (64 q vectors) and
// streams the K and V pages once per block: pass 1 over the K pages for the row maxima and sums
// (kept per warp, combined once), pass 2 over (K, V) page pairs - scores recomputed bit for bit,
// weights bf16(exp(s - M) / L) final before P.V, as in the one-row forms.  Scores come from
// mma.sync with the q vectors as the B operand (bf16 hi + lo halves: f32-accurate q), the weights
// go through shared memory to become the A operand of P.V.  Keys past a row's own position are
// masked; pages past the block's last row are never fetched.  All rows of the body must already be
// in the cache (attn_append_kernel).
// ------------------------------------------------------------------------------------------------
constexpr int kPfRows = 16;                   // rows (positions) per CTA
constexpr int kPfQ = kPfRows * 4;             // q vectors per CTA; n = row * 4 + head
constexpr int kPfQLd = 264;                   // bf16 row stride of a q tile (528 B: conflict-free ldmatrix)
constexpr int kPfPLd = 72;                    // bf16 row stride of a weight tile (144 B)
constexpr int kPfRing = 3;
constexpr size_t kPfSmem = 1024 + (size_t)kPfRing * kTileBytes + 2 * (size_t)kPfQ * kPfQLd * 2 +
                           2 * (size_t)kPfQ * kPfPLd * 2 + 4 * kPfQ * 2 * 4;

__global__ void __launch_bounds__(kTmaThreads, 1)
attn_prefill_kernel(AttnParams p, const __grid_constant__ CUtensorMap kmap, const __grid_constant__ CUtensorMap vmap) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) unsigned long long bars[2 * kPfRing];
    if (threadIdx.x == 0) { prefetch_tensormap(&kmap); prefetch_tensormap(&vmap); }
    pdl_wait();
    if (p.status != nullptr && *p.status != 0) return;

    const uint32_t ring = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* base_ptr = smem_raw + (ring - smem_u32(smem_raw));
    uint16_t* Qhi = reinterpret_cast<uint16_t*>(base_ptr + kPfRing * kTileBytes);     // [64][264]
    uint16_t* Qlo = Qhi + kPfQ * kPfQLd;
    uint16_t* P_s = Qlo + kPfQ * kPfQLd;                                              // [2][64][72]
    float* stat_s = reinterpret_cast<float*>(P_s + 2 * kPfQ * kPfPLd);                // [4 m-tiles][64][2]
    const uint32_t full0 = smem_u32(&bars[0]), empty0 = smem_u32(&bars[kPfRing]);

    const int lane_id = blockIdx.x, kvh = blockIdx.y, t0 = blockIdx.z * kPfRows;
    const int tid = threadIdx.x, warp = tid >> 5, ln = tid & 31;
    const int g = ln >> 2, t = ln & 3;
    const int cap = p.pages_per_lane * kKvPage;
    const int slot0 = p.slot[lane_id] > 0 ? p.slot[lane_id] : 0;   // position of the body's first row (never negative)
    const int rope0 = p.rope_pos[lane_id];
    const int rows_here = (p.T - t0) < kPfRows ? (p.T - t0) : kPfRows;
    int last = slot0 + t0 + rows_here - 1;                  // last key position any row of the block sees
    if (last >= cap) last = cap - 1;
    const int P = last / kKvPage + 1;                       // pages the block reads
    const int* table = p.page_table + (size_t)lane_id * p.table_lane_stride;

    if (tid == 0) {
        for (int b = 0; b < kPfRing; ++b) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;\n" ::"r"(full0 + 8 * b) : "memory");
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 8;\n" ::"r"(empty0 + 8 * b) : "memory");
        }
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    __syncthreads();

    if (warp == 8) {
        // ---- producer: K pages 0..P-1, then (K, V) of page 0, of page 1, ... ---------------------
        if (ln == 0) {
            bool ok = true;
            for (int i = 0; i < 3 * P && ok; ++i) {
                const int b = i % kPfRing;
                ok = mbar_wait(empty0 + 8 * b, ((i / kPfRing) & 1) ^ 1);
                if (!ok) break;
                const int page_i = i < P ? i : ((i - P) >> 1);
                const bool is_v = i >= P && ((i - P) & 1);
                const CUtensorMap* map = is_v ? &vmap : &kmap;
                const uint32_t dst = ring + b * kTileBytes;
                const int r0 = table[page_i] * (kKvHeads * kKvPage) + kvh * kKvPage;
                asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(full0 + 8 * b), "r"(kTileBytes) : "memory");
#pragma unroll
                for (int cb = 0; cb < 4; ++cb)
                    asm volatile(
                        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n"
                        ::"r"(dst + cb * 8192), "l"(reinterpret_cast<uint64_t>(map)), "r"(full0 + 8 * b), "r"(cb * 64), "r"(r0) : "memory");
            }
            if (!ok && p.status != nullptr) atomicExch(p.status, 5);
        }
        return;
    }

    // ---- q vectors of the block: norm + rope in f32, split into bf16 hi + lo ----------------------
    for (int n = warp * 8; n < warp * 8 + 8; ++n) {
        const int r = n >> 2, head = kvh * 4 + (n & 3);
        uint4 hi4 = make_uint4(0, 0, 0, 0), lo4 = make_uint4(0, 0, 0, 0);
        if (r < rows_here) {                                   // warp-uniform
            const uint16_t* pr = p.proj + ((size_t)lane_id * p.T + t0 + r) * kAttnProjN;
            float x[8], h8[8], l8[8];
            unpack8(*reinterpret_cast<const uint4*>(pr + head * 2 * kHeadDim + 8 * ln), x);
            head_norm_rope(x, p.q_norm, ln, rope0 + t0 + r, p.inv_freq);
#pragma unroll
            for (int e = 0; e < 8; ++e) { h8[e] = bfround(x[e]); l8[e] = x[e] - h8[e]; }
            hi4 = pack8(h8);
            lo4 = pack8(l8);
        }
        *reinterpret_cast<uint4*>(Qhi + n * kPfQLd + 8 * ln) = hi4;
        *reinterpret_cast<uint4*>(Qlo + n * kPfQLd + 8 * ln) = lo4;
    }
    asm volatile("bar.sync 1, 256;\n" ::: "memory");

    const int mt = warp & 3, nh = warp >> 2;               // 16-position m-tile, 32-q-vector half
    bool ok = true;
    // scores of this warp's (m-tile, q half) for the page in ring slot `tile`: acc[nt][0..3]
    auto scores = [&](uint32_t tile, float (&acc)[4][4]) {
#pragma unroll
        for (int nt = 0; nt < 4; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[nt][e] = 0.f;
#pragma unroll 4
        for (int ks = 0; ks < 16; ++ks) {
            uint32_t a[4];
            ldsm_x4(a, tile + tile_off(mt * 16 + (ln & 15), ks * 2 + (ln >> 4)));
            const int blk = ln >> 3, rr = ln & 7;
#pragma unroll
            for (int np = 0; np < 2; ++np) {
                const int n = nh * 32 + (np * 2 + (blk >> 1)) * 8 + rr;
                const uint32_t off = (uint32_t)(n * kPfQLd + ks * 16 + (blk & 1) * 8) * 2;
                uint32_t bh[4], bl[4];
                ldsm_x4(bh, smem_u32(Qhi) + off);
                ldsm_x4(bl, smem_u32(Qlo) + off);
                mma_bf16(acc[2 * np], a[0], a[1], a[2], a[3], bh[0], bh[1]);
                mma_bf16(acc[2 * np], a[0], a[1], a[2], a[3], bl[0], bl[1]);
                mma_bf16(acc[2 * np + 1], a[0], a[1], a[2], a[3], bh[2], bh[3]);
                mma_bf16(acc[2 * np + 1], a[0], a[1], a[2], a[3], bl[2], bl[3]);
            }
        }
    };
    // key position limit of the q vector in column (nt, e & 1): its own row's position; -1 = no row
    auto limit_of = [&](int nt, int e) {
        const int n = nh * 32 + nt * 8 + 2 * t + (e & 1);
        const int r = n >> 2;
        return r < rows_here ? slot0 + t0 + r : -1;
    };

    // ---- pass 1: per-column running max and sum over this warp's positions ------------------------
    float M[8], L[8];
#pragma unroll
    for (int c8 = 0; c8 < 8; ++c8) { M[c8] = -INFINITY; L[c8] = 0.f; }
    for (int j = 0; j < P; ++j) {
        const int b = j % kPfRing;
        if (ok) ok = mbar_wait(full0 + 8 * b, (j / kPfRing) & 1);
        float acc[4][4];
        scores(ring + b * kTileBytes, acc);
        __syncwarp();
        if (ln == 0) mbar_arrive(empty0 + 8 * b);
        const int pos_lo = j * kKvPage + mt * 16 + g;
#pragma unroll
        for (int nt = 0; nt < 4; ++nt)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int lim = limit_of(nt, e);
                const float s0 = pos_lo <= lim ? acc[nt][e] * 0.0625f : -INFINITY;
                const float s1 = pos_lo + 8 <= lim ? acc[nt][2 + e] * 0.0625f : -INFINITY;
                float pm = fmaxf(s0, s1);
                pm = fmaxf(pm, __shfl_xor_sync(0xffffffffu, pm, 4));
                pm = fmaxf(pm, __shfl_xor_sync(0xffffffffu, pm, 8));
                pm = fmaxf(pm, __shfl_xor_sync(0xffffffffu, pm, 16));
                const int c8 = nt * 2 + e;
                const float Mn = fmaxf(M[c8], pm);
                float add = 0.f;
                if (Mn > -INFINITY) add = (s0 > -INFINITY ? expf(s0 - Mn) : 0.f) + (s1 > -INFINITY ? expf(s1 - Mn) : 0.f);
                add += __shfl_xor_sync(0xffffffffu, add, 4);
                add += __shfl_xor_sync(0xffffffffu, add, 8);
                add += __shfl_xor_sync(0xffffffffu, add, 16);
                if (Mn > -INFINITY) L[c8] = L[c8] * (M[c8] > -INFINITY ? expf(M[c8] - Mn) : 0.f) + add;
                M[c8] = Mn;
            }
    }
    if (g == 0) {
#pragma unroll
        for (int c8 = 0; c8 < 8; ++c8) {
            const int n = nh * 32 + (c8 >> 1) * 8 + 2 * t + (c8 & 1);
            stat_s[(mt * kPfQ + n) * 2] = M[c8];
            stat_s[(mt * kPfQ + n) * 2 + 1] = L[c8];
        }
    }
    asm volatile("bar.sync 1, 256;\n" ::: "memory");
#pragma unroll
    for (int c8 = 0; c8 < 8; ++c8) {
        const int n = nh * 32 + (c8 >> 1) * 8 + 2 * t + (c8 & 1);
        float Mf = -INFINITY;
#pragma unroll
        for (int m4 = 0; m4 < 4; ++m4) Mf = fmaxf(Mf, stat_s[(m4 * kPfQ + n) * 2]);
        float Lf = 0.f;
#pragma unroll
        for (int m4 = 0; m4 < 4; ++m4) {
            const float mm = stat_s[(m4 * kPfQ + n) * 2], ll = stat_s[(m4 * kPfQ + n) * 2 + 1];
            if (ll > 0.f) Lf += ll * expf(mm - Mf);
        }
        M[c8] = Mf;
        L[c8] = Lf;
    }

    // ---- pass 2: weights of a page -> shared memory -> P.V ---------------------------------------
    float O[4][4][4];
#pragma unroll
    for (int mm = 0; mm < 4; ++mm)
#pragma unroll
        for (int nt = 0; nt < 4; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) O[mm][nt][e] = 0.f;
    for (int j = 0; j < P; ++j) {
        const int ik = P + 2 * j, iv = ik + 1;
        const int bk = ik % kPfRing, bv = iv % kPfRing;
        if (ok) ok = mbar_wait(full0 + 8 * bk, (ik / kPfRing) & 1);
        float acc[4][4];
        scores(ring + bk * kTileBytes, acc);
        __syncwarp();
        if (ln == 0) mbar_arrive(empty0 + 8 * bk);
        uint16_t* Pw = P_s + (j & 1) * kPfQ * kPfPLd;
        const int pos_lo = j * kKvPage + mt * 16 + g;
#pragma unroll
        for (int nt = 0; nt < 4; ++nt)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int lim = limit_of(nt, e);
                const int c8 = nt * 2 + e;
                const int n = nh * 32 + nt * 8 + 2 * t + e;
                const float w0 = pos_lo <= lim ? __fdiv_rn(expf(acc[nt][e] * 0.0625f - M[c8]), L[c8]) : 0.f;
                const float w1 = pos_lo + 8 <= lim ? __fdiv_rn(expf(acc[nt][2 + e] * 0.0625f - M[c8]), L[c8]) : 0.f;
                Pw[n * kPfPLd + mt * 16 + g] = f2bf(w0);
                Pw[n * kPfPLd + mt * 16 + g + 8] = f2bf(w1);
            }
        asm volatile("bar.sync 1, 256;\n" ::: "memory");
        if (ok) ok = mbar_wait(full0 + 8 * bv, (iv / kPfRing) & 1);
        const uint32_t vt = ring + bv * kTileBytes;
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
            uint32_t bfr[2][4];
#pragma unroll
            for (int np = 0; np < 2; ++np) {
                const int pos = ks * 16 + (ln & 7) + ((ln >> 3) & 1) * 8;
                ldsm_x4_trans(bfr[np], vt + tile_off(pos, warp * 4 + np * 2 + (ln >> 4)));
            }
#pragma unroll
            for (int mm = 0; mm < 4; ++mm) {
                uint32_t a[4];
                ldsm_x4(a, smem_u32(Pw) + (uint32_t)((mm * 16 + (ln & 15)) * kPfPLd + ks * 16 + (ln >> 4) * 8) * 2);
#pragma unroll
                for (int np = 0; np < 2; ++np) {
                    mma_bf16(O[mm][2 * np], a[0], a[1], a[2], a[3], bfr[np][0], bfr[np][1]);
                    mma_bf16(O[mm][2 * np + 1], a[0], a[1], a[2], a[3], bfr[np][2], bfr[np][3]);
                }
            }
        }
        __syncwarp();
        if (ln == 0) mbar_arrive(empty0 + 8 * bv);
    }
    if (!ok) {
        if (ln == 0 && p.status != nullptr) atomicExch(p.status, 6);
        return;
    }

    // ---- epilogue: round, apply the bf16 sigmoid gate ---------------------------------------------
#pragma unroll
    for (int mm = 0; mm < 4; ++mm)
#pragma unroll
        for (int hrow = 0; hrow < 2; ++hrow) {
            const int n = mm * 16 + g + hrow * 8;
            const int r = n >> 2, head = kvh * 4 + (n & 3);
            if (r >= rows_here) continue;
            const size_t row = (size_t)lane_id * p.T + t0 + r;
            const uint16_t* pr = p.proj + row * kAttnProjN;
#pragma unroll
            for (int nt = 0; nt < 4; ++nt) {
                const int dd = warp * 32 + nt * 8 + 2 * t;
                const uint32_t gw = *reinterpret_cast<const uint32_t*>(pr + head * 2 * kHeadDim + kHeadDim + dd);
                const float o0 = bfround(O[mm][nt][2 * hrow]) * bfround(sigmoid_acc(lo_bf(gw)));
                const float o1 = bfround(O[mm][nt][2 * hrow + 1]) * bfround(sigmoid_acc(hi_bf(gw)));
                *reinterpret_cast<uint32_t*>(p.out + row * (kQHeads * kHeadDim) + head * kHeadDim + dd) = pack_bf2(o0, o1);
            }
        }
}

size_t attn_tma_smem(int ctx_pad) {
    return 1024 + (size_t)kRing * kTileBytes + 4 * kHeadDim * 4 + (size_t)8 * ctx_pad * 4 + (size_t)4 * ctx_pad * 2;
}

}  // namespace

// Tensor map of a K or V page pool seen as a matrix [n_pages * 128 rows][256] bf16, box 64 x 64.
bool attn_make_pool_map(void* map_out, const uint16_t* pool, long long n_pages) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (fn == nullptr || n_pages <= 0) return false;
    cuuint64_t dims[2] = {(cuuint64_t)kHeadDim, (cuuint64_t)n_pages * kKvHeads * kKvPage};
    cuuint64_t strides[1] = {(cuuint64_t)kHeadDim * 2};
    cuuint32_t box[2] = {64, 64};
    cuuint32_t elem[2] = {1, 1};
    return fn(static_cast<CUtensorMap*>(map_out), CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<uint16_t*>(pool),
              dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
              CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

static size_t attn_smem_bytes(int ctx_pad) {
    return (size_t)(4 * kHeadDim + 8 * 4 * kHeadDim + 4 * ctx_pad) * sizeof(float);
}

cudaError_t attn_init() {
    const int max_bytes = (int)attn_smem_bytes(kAttnMaxCtx);
    cudaError_t e = cudaFuncSetAttribute(attn_decode_kernel<true>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, max_bytes);
    if (e != cudaSuccess) return e;
    e = cudaFuncSetAttribute(attn_decode_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_bytes);
    if (e != cudaSuccess) return e;
    const int tma_bytes = (int)attn_tma_smem(kAttnTmaMaxCtx);
    e = cudaFuncSetAttribute(attn_tma_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, tma_bytes);
    if (e != cudaSuccess) return e;
    e = cudaFuncSetAttribute(attn_prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kPfSmem);
    if (e != cudaSuccess) return e;
    e = cudaFuncSetAttribute(attn_cluster_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, tma_bytes);
    if (e != cudaSuccess) return e;
    e = cudaFuncSetAttribute(attn_cluster_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, tma_bytes);
    if (e != cudaSuccess) return e;
    return cudaFuncSetAttribute(attn_tma_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, tma_bytes);
}

cudaError_t launch_attn(const AttnParams& p, cudaStream_t st) {
    if (p.lanes <= 0 || p.T <= 0 || p.max_ctx <= 0 || p.max_ctx > kAttnMaxCtx) return cudaErrorInvalidValue;
    const int ctx_pad = (p.max_ctx + 31) & ~31;
    const int rows = p.lanes * p.T;
    const dim3 grid(rows, kKvHeads);
    if (p.T > 1) {
        cudaError_t e = launch_k(attn_append_kernel, grid, dim3(64), 0, st, p);
        if (e != cudaSuccess) return e;
    }
    // prompt bodies: blocks of 16 rows share one pass over the lane's pages
    static int prefill_mode = -1;
    if (prefill_mode < 0) {
        const char* env = std::getenv("Q35_ATTN_PREFILL");
        prefill_mode = (env != nullptr && env[0] == '0') ? 0 : 1;
    }
    if (prefill_mode && p.T >= kPfRows) {
        CUtensorMap kmap, vmap;
        if (p.kmap != nullptr && p.vmap != nullptr) {
            kmap = *static_cast<const CUtensorMap*>(p.kmap);
            vmap = *static_cast<const CUtensorMap*>(p.vmap);
        } else if (!attn_make_pool_map(&kmap, p.kpool, p.n_pages) || !attn_make_pool_map(&vmap, p.vpool, p.n_pages)) {
            return cudaErrorInvalidValue;
        }
        return launch_k(attn_prefill_kernel, dim3(p.lanes, kKvHeads, (p.T + kPfRows - 1) / kPfRows), dim3(kTmaThreads),
                        kPfSmem, st, p, kmap, vmap);
    }
    if (ctx_pad <= kAttnTmaMaxCtx) {
        CUtensorMap kmap, vmap;
        if (p.kmap != nullptr && p.vmap != nullptr) {
            kmap = *static_cast<const CUtensorMap*>(p.kmap);
            vmap = *static_cast<const CUtensorMap*>(p.vmap);
        } else if (!attn_make_pool_map(&kmap, p.kpool, p.n_pages) || !attn_make_pool_map(&vmap, p.vpool, p.n_pages)) {
            return cudaErrorInvalidValue;
        }
        const int pad64 = (p.max_ctx + 63) & ~63;           // whole pages
        const size_t smem = attn_tma_smem(pad64);
        // few lanes: a cluster of CTAs per (row, kv head) splits the context by pages.  The cluster
        // size follows the LANE count, not the row count, so a one-token step and a multi-token
        // verify body of the same lanes sum in the same order.
        static int cluster_mode = -1;
        if (cluster_mode < 0) {
            const char* env = std::getenv("Q35_ATTN_CLUSTER");
            cluster_mode = (env != nullptr && env[0] == '0') ? 0 : 1;
        }
        int cs = 1;
        if (cluster_mode) {
            cs = p.lanes <= 8 ? 8 : (p.lanes <= 32 ? 4 : 1);      // measured: no gain from 64 lanes up
            if (p.T > 4) cs = 1;                                 // prompt bodies bring their own parallelism
            static int forced = -1;                      // tuning knob: Q35_ATTN_CS = 1, 2, 4 or 8
            if (forced < 0) {
                const char* env = std::getenv("Q35_ATTN_CS");
                forced = env != nullptr ? std::atoi(env) : 0;
                if (forced != 1 && forced != 2 && forced != 4 && forced != 8) forced = 0;
            }
            if (forced) cs = forced;
            while (cs > pad64 / kKvPage) cs >>= 1;
        }
        if (cs > 1) {
            cudaLaunchConfig_t cfg{};
            cfg.gridDim = dim3(rows, kKvHeads, cs);
            cfg.blockDim = dim3(kTmaThreads);
            const int lpad = ((pad64 / kKvPage + cs - 1) / cs) * kKvPage;      // positions a CTA of the cluster can own
            cfg.dynamicSmemBytes = attn_tma_smem(lpad);
            cfg.stream = st;
            cudaLaunchAttribute at[2];
            at[0].id = cudaLaunchAttributeClusterDimension;
            at[0].val.clusterDim.x = 1;
            at[0].val.clusterDim.y = 1;
            at[0].val.clusterDim.z = cs;
            at[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
            at[1].val.programmaticStreamSerializationAllowed = 1;
            cfg.attrs = at;
            cfg.numAttrs = pdl_enabled() ? 2 : 1;
            if (p.T == 1) return cudaLaunchKernelEx(&cfg, attn_cluster_kernel<true>, p, pad64, lpad, cs, kmap, vmap);
            return cudaLaunchKernelEx(&cfg, attn_cluster_kernel<false>, p, pad64, lpad, cs, kmap, vmap);
        }
        if (p.T == 1) return launch_k(attn_tma_kernel<true>, grid, dim3(kTmaThreads), smem, st, p, pad64, kmap, vmap);
        return launch_k(attn_tma_kernel<false>, grid, dim3(kTmaThreads), smem, st, p, pad64, kmap, vmap);
    }
    const size_t smem = attn_smem_bytes(ctx_pad);
    if (p.T == 1) return launch_k(attn_decode_kernel<true>, grid, dim3(256), smem, st, p, ctx_pad);
    return launch_k(attn_decode_kernel<false>, grid, dim3(256), smem, st, p, ctx_pad);
}

}  // namespace q35
