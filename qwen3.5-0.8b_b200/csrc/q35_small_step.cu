// One persistent kernel per decode step for few lanes (<= 16).
//
// At few lanes the step moves ~1.5 GB of weights through 172 small dependent kernels and is bound
// by their launch + DRAM-latency chain, not by bandwidth.  Here ONE kernel with one CTA per SM walks
// the whole step: embedding -> 24 x (in-proj, mixer, out-proj, gate/up, down) -> head + argmax.
// Phases are separated by grid barriers (an atomic counter in global memory, bounded polling), and
// before working on a phase every CTA asks L2 (cp.async.bulk.prefetch.L2) for the weight rows it
// will need two phases later, so HBM keeps streaming weights through the barriers and every
// phase's loads hit L2.  Residual add + RMSNorm ride in the prologue of the phase that consumes
// them (recomputed per CTA: <= 16 rows).  Arithmetic and rounding points are those of the
// multi-kernel path (q35_glue / q35_gemm / q35_gdn / q35_attn); attention over several CTAs uses the
// block-wise (max, sum)-rescaled softmax, which the reference accepts as the same contract
// (speccheck/specimpl.py:350-372).
//
// Replaces, for one to sixteen requests, the reference's 340-launch decode_step
// (engine/decode_step.cpp:448-1354).
//
// MEASURED (B200, 512-token context): 1.09 ms/step at 1 lane and 1.52 ms at 16 lanes, against 1.01 and
// 1.18 ms for the 172-kernel CUDA-graph path.  The phase clock (q35_small_step_trace) shows ~1.9 us per
// grid barrier and 3.5-9 us of work per phase that does not shrink when the weights are already in
// registers: every phase pays two or three dependent L2 round trips (inputs written by other SMs,
// barrier atomics), which on this two-die part cost more than a kernel boundary saves.  The engine
// therefore takes this kernel only when Q35_SMALL_STEP=1.
#include "q35_common.cuh"
#include "q35_async.cuh"

namespace q35 {

namespace {

constexpr int kThreads = 256;
constexpr int XLD1 = kHidden + 8;          // padded bf16 row strides: conflict-free 16-byte reads
constexpr int XLD2 = 2048 + 8;
constexpr int XLD3 = kFF + 8;
constexpr size_t kSmallSmem = (size_t)16 * XLD3 * 2;      // largest x tile: 16 rows of the SwiGLU act

__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint16_t swiglu_bf16(float gate_acc, float up_acc) {
    const float g = bfround(gate_acc);
    const float u = bfround(up_acc);
    const float s = bfround(silu_acc(g));
    return f2bf(s * u);
}
// ask L2 for `bytes` (multiple of 16) starting at p (16-byte aligned); fire and forget
// bf16 value written by another CTA earlier in this launch: read through L2, never a stale L1 line
__device__ __forceinline__ float ldcg_bf(const uint16_t* p) { return bf2f(__ldcg(p)); }
__device__ __forceinline__ void l2_prefetch(const void* p, uint32_t bytes) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;\n" ::"l"(p), "r"(bytes) : "memory");
}

// Grid barrier: every CTA adds one to a counter that only grows during a launch and waits until it
// reaches `target`.  Bounded: after ~1 s of polling the CTA raises the status word and the caller
// leaves the kernel.  Returns false on expiry.
__device__ __forceinline__ bool grid_barrier(unsigned* counter, unsigned target, int* status, int* abort_s) {
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        atomicAdd(counter, 1u);
        const unsigned long long t0 = global_ns();
        for (;;) {
            unsigned v;
            asm volatile("ld.acquire.gpu.global.u32 %0, [%1];\n" : "=r"(v) : "l"(counter) : "memory");
            if (v >= target) break;
            if (global_ns() - t0 > 1000000000ull) {
                *abort_s = 1;
                if (status != nullptr) atomicExch(status, 7);
                break;
            }
        }
        __threadfence();
    }
    __syncthreads();
    return *abort_s == 0;
}

// x rows -> shared memory as bf16, optionally through  sum = bf16(src + delta); x = RMSNorm_zc(sum; w).
// Warp w takes rows w and w + 8.  Rows >= M are zero.  CTA 0 may store the sum / the normed rows.
// src row r is table[ids[r]] when ids != null, else src + r * 1024.
__device__ __forceinline__ void norm_rows_to_smem(uint16_t* xs, const uint16_t* __restrict__ src,
                                                  const int* __restrict__ ids, const uint16_t* __restrict__ table,
                                                  int vocab, const uint16_t* __restrict__ delta,
                                                  const uint16_t* __restrict__ w, int M, uint16_t* sum_out,
                                                  uint16_t* normed_out) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int r = warp + 8 * half;
        uint4* dst = reinterpret_cast<uint4*>(xs + r * XLD1);
        if (r >= M) {
#pragma unroll
            for (int c = 0; c < 4; ++c) dst[c * 32 + lane] = make_uint4(0, 0, 0, 0);
            continue;
        }
        const uint16_t* row;
        if (ids != nullptr) {
            int id = ids[r];
            id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
            row = table + (size_t)id * kHidden;
        } else {
            row = src + (size_t)r * kHidden;
        }
        float v[32];
        float ss = 0.f;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            const int off = c * 256 + lane * 8;
            const uint4 a = __ldcg(reinterpret_cast<const uint4*>(row + off));
            const uint32_t aw[4] = {a.x, a.y, a.z, a.w};
            uint32_t dw[4] = {0, 0, 0, 0};
            if (delta != nullptr) {
                const uint4 d = __ldcg(reinterpret_cast<const uint4*>(delta + (size_t)r * kHidden + off));
                dw[0] = d.x; dw[1] = d.y; dw[2] = d.z; dw[3] = d.w;
            }
            uint32_t sw[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                float lo = lo_bf(aw[j]), hi = hi_bf(aw[j]);
                if (delta != nullptr) {
                    lo = bfround(lo + lo_bf(dw[j]));
                    hi = bfround(hi + hi_bf(dw[j]));
                }
                v[c * 8 + 2 * j] = lo;
                v[c * 8 + 2 * j + 1] = hi;
                ss += lo * lo + hi * hi;
                sw[j] = pack_bf2(lo, hi);
            }
            if (sum_out != nullptr)
                *reinterpret_cast<uint4*>(sum_out + (size_t)r * kHidden + off) = make_uint4(sw[0], sw[1], sw[2], sw[3]);
        }
        ss = warp_sum(ss);
        const float inv = rsqrt_acc(ss * (1.0f / kHidden) + kEps);
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            const int off = c * 256 + lane * 8;
            const uint4 wn = __ldg(reinterpret_cast<const uint4*>(w + off));
            const uint32_t ww[4] = {wn.x, wn.y, wn.z, wn.w};
            uint32_t o[4];
#pragma unroll
            for (int j = 0; j < 4; ++j)
                o[j] = pack_bf2(__fmul_rn(__fmul_rn(v[c * 8 + 2 * j], inv), 1.0f + lo_bf(ww[j])),
                                __fmul_rn(__fmul_rn(v[c * 8 + 2 * j + 1], inv), 1.0f + hi_bf(ww[j])));
            const uint4 ov = make_uint4(o[0], o[1], o[2], o[3]);
            dst[c * 32 + lane] = ov;
            if (normed_out != nullptr) *reinterpret_cast<uint4*>(normed_out + (size_t)r * kHidden + off) = ov;
        }
    }
}

// plain copy of M rows of `width` bf16 from global into padded shared rows (rows >= M zeroed)
__device__ __forceinline__ void rows_to_smem(uint16_t* xs, int xld, const uint16_t* __restrict__ src, int width, int M) {
    const int chunks = width / 8;
    for (int i = threadIdx.x; i < 16 * chunks; i += kThreads) {
        const int r = i / chunks, c = i % chunks;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (r < M) v = __ldcg(reinterpret_cast<const uint4*>(src + (size_t)r * width + c * 8));
        *reinterpret_cast<uint4*>(xs + r * xld + c * 8) = v;
    }
}

// ---- few-row GEMV pieces.  Weight registers are loaded BEFORE the grid barrier that precedes the
// phase (weights depend on nothing), so the loads complete while the CTA waits at the barrier. -----
// One warp: 8 weight rows n0..n0+7, whole K = 1024, in two halves of 16 chunks of 32 k.
__device__ __forceinline__ void wg_load_half(uint4 (&w)[16], const uint16_t* __restrict__ W, int n0, int N, int half) {
    const int lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    int n = n0 + g;
    n = n < N ? n : N - 1;
    const uint16_t* wrow = W + (size_t)n * kHidden + t * 8 + half * 512;
#pragma unroll
    for (int c = 0; c < 16; ++c) w[c] = __ldg(reinterpret_cast<const uint4*>(wrow + c * 32));
}
// acc[0..3] = (row g, cols 2t, 2t+1), (row g+8, cols 2t, 2t+1) against the 16 x 1024 x tile in smem
__device__ __forceinline__ void wg_compute(const uint16_t* xs, const uint4 (&w0)[16], const uint4 (&w1)[16], float (&acc)[4]) {
    const int lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    // four independent accumulator chains: 64 dependent MMAs on one accumulator would be all latency
    float a4[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) a4[i][j] = 0.f;
#pragma unroll
    for (int c = 0; c < 16; ++c) {
        const int k = c * 32 + t * 8;
        const uint4 xl = *reinterpret_cast<const uint4*>(xs + g * XLD1 + k);
        const uint4 xh = *reinterpret_cast<const uint4*>(xs + (g + 8) * XLD1 + k);
        mma16816(a4[c & 1], xl.x, xh.x, xl.y, xh.y, w0[c].x, w0[c].y);
        mma16816(a4[2 + (c & 1)], xl.z, xh.z, xl.w, xh.w, w0[c].z, w0[c].w);
    }
#pragma unroll
    for (int c = 0; c < 16; ++c) {
        const int k = 512 + c * 32 + t * 8;
        const uint4 xl = *reinterpret_cast<const uint4*>(xs + g * XLD1 + k);
        const uint4 xh = *reinterpret_cast<const uint4*>(xs + (g + 8) * XLD1 + k);
        mma16816(a4[c & 1], xl.x, xh.x, xl.y, xh.y, w1[c].x, w1[c].y);
        mma16816(a4[2 + (c & 1)], xl.z, xh.z, xl.w, xh.w, w1[c].z, w1[c].w);
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[j] = (a4[0][j] + a4[1][j]) + (a4[2][j] + a4[3][j]);
}

// One CTA: 8 weight rows n0..n0+7, K split over the 8 warps (K/8/32 <= 14 chunks per thread).
template <int K>
__device__ __forceinline__ void cu_load(uint4 (&w)[16], const uint16_t* __restrict__ W, int n0, int N) {
    constexpr int KW = K / 8, CH = KW / 32;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    int n = n0 + g;
    n = n < N ? n : N - 1;
    const uint16_t* wrow = W + (size_t)n * K + warp * KW + t * 8;
#pragma unroll
    for (int c = 0; c < CH; ++c) w[c] = __ldg(reinterpret_cast<const uint4*>(wrow + c * 32));
}
// partial sums reduced through `red` ([8][16][8] floats); out[row][n0 + col] = bf16(sum) for row < M
template <int K, int XLD>
__device__ __forceinline__ void cu_compute(const uint16_t* xs, const uint4 (&w)[16], int n0, int N, int M, float* red,
                                           uint16_t* __restrict__ out) {
    constexpr int KW = K / 8, CH = KW / 32;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int kbase = warp * KW + t * 8;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int c = 0; c < CH; ++c) {
        const uint4 xl = *reinterpret_cast<const uint4*>(xs + g * XLD + kbase + c * 32);
        const uint4 xh = *reinterpret_cast<const uint4*>(xs + (g + 8) * XLD + kbase + c * 32);
        mma16816(acc, xl.x, xh.x, xl.y, xh.y, w[c].x, w[c].y);
        mma16816(acc, xl.z, xh.z, xl.w, xh.w, w[c].z, w[c].w);
    }
    float* r = red + warp * 128;
    r[g * 8 + 2 * t] = acc[0]; r[g * 8 + 2 * t + 1] = acc[1];
    r[(g + 8) * 8 + 2 * t] = acc[2]; r[(g + 8) * 8 + 2 * t + 1] = acc[3];
    __syncthreads();
    if (threadIdx.x < 128) {
        const int row = threadIdx.x >> 3, col = threadIdx.x & 7;
        float s = 0.f;
#pragma unroll
        for (int w8 = 0; w8 < 8; ++w8) s += red[w8 * 128 + threadIdx.x];
        if (row < M && n0 + col < N) out[(size_t)row * N + n0 + col] = f2bf(s);
    }
    __syncthreads();
}

// ---- GDN: one (lane, head) item by the whole CTA, one token, state tile in registers -------------
// Same arithmetic as gdn_step_kernel (q35_gdn.cu); plain loads (the tile was prefetched into L2).
struct GdnShared {
    float q[128], k[128], v[128];
    __align__(16) float red_r[8][128];
    __align__(16) float red_o[8][128];
    float ssum[4][2];
    float osum[4];
};

__device__ __forceinline__ void gdn_item(GdnShared& sh, const uint16_t* __restrict__ pr, const uint16_t* __restrict__ conv_w,
                                         const uint16_t* __restrict__ A_log, const uint16_t* __restrict__ dt_bias,
                                         const uint16_t* __restrict__ norm_w, float* __restrict__ S_tile,
                                         uint16_t* __restrict__ win, int h, uint16_t* __restrict__ y_row) {
    constexpr int kOffZ = 6144, kOffB = 8192, kOffA = 8208;
    const int tid = threadIdx.x, warp = tid >> 5, ln = tid & 31;
    float4 s[16];
    {
        const float4* Sp = reinterpret_cast<const float4*>(S_tile);
#pragma unroll
        for (int r = 0; r < 16; ++r) s[r] = __ldcg(Sp + (warp * 16 + r) * 32 + ln);
    }
    const float negA = -expf(bf2f(A_log[h]));
    const float dtb = bf2f(dt_bias[h]);
    const float b_in = ldcg_bf(pr + kOffB + h), a_in = ldcg_bf(pr + kOffA + h);
    const float z_in = tid < 128 ? ldcg_bf(pr + kOffZ + h * 128 + tid) : 0.f;
    const float nw_in = tid < 128 ? bf2f(norm_w[tid]) : 0.f;
    const float q_scale = 0.08838834764831845f;
    float wnew[3][3];
    int ch[3] = {0, 0, 0};
    if (tid < 128) {
        float u[3];
#pragma unroll
        for (int kind = 0; kind < 3; ++kind) {
            ch[kind] = kind * 2048 + h * 128 + tid;
            const uint2 tw = __ldg(reinterpret_cast<const uint2*>(conv_w + (size_t)ch[kind] * 4));
            const float tap[4] = {lo_bf(tw.x), hi_bf(tw.x), lo_bf(tw.y), hi_bf(tw.y)};
            float w[3];
#pragma unroll
            for (int j = 0; j < 3; ++j) w[j] = bf2f(win[j * kConvCh + ch[kind]]);
            const float raw = ldcg_bf(pr + ch[kind]);
            float acc = __fmul_rn(w[0], tap[0]);
            acc = __fadd_rn(acc, __fmul_rn(w[1], tap[1]));
            acc = __fadd_rn(acc, __fmul_rn(w[2], tap[2]));
            acc = __fadd_rn(acc, __fmul_rn(raw, tap[3]));
            u[kind] = bfround(silu_acc(bfround(acc)));
            wnew[kind][0] = w[1]; wnew[kind][1] = w[2]; wnew[kind][2] = raw;
        }
        sh.q[tid] = u[0]; sh.k[tid] = u[1]; sh.v[tid] = u[2];
        const float qq = warp_sum(u[0] * u[0]);
        const float kk = warp_sum(u[1] * u[1]);
        if (ln == 0) { sh.ssum[warp][0] = qq; sh.ssum[warp][1] = kk; }
    }
    __syncthreads();
    const float qinv = rsqrt_acc(sh.ssum[0][0] + sh.ssum[1][0] + sh.ssum[2][0] + sh.ssum[3][0] + 1e-6f);
    const float kinv = rsqrt_acc(sh.ssum[0][1] + sh.ssum[1][1] + sh.ssum[2][1] + sh.ssum[3][1] + 1e-6f);
    const float beta = sigmoid_acc(b_in);
    const float sp_in = a_in + dtb;
    const float sp = sp_in > 20.0f ? sp_in : log1pf(expf(sp_in));
    const float gamma = expf(__fmul_rn(negA, sp));

    float4 pr4 = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int r = 0; r < 16; ++r) {
        const float kh = __fmul_rn(sh.k[warp * 16 + r], kinv);
        s[r].x = __fmul_rn(s[r].x, gamma); s[r].y = __fmul_rn(s[r].y, gamma);
        s[r].z = __fmul_rn(s[r].z, gamma); s[r].w = __fmul_rn(s[r].w, gamma);
        pr4.x += s[r].x * kh; pr4.y += s[r].y * kh; pr4.z += s[r].z * kh; pr4.w += s[r].w * kh;
    }
    *reinterpret_cast<float4*>(&sh.red_r[warp][4 * ln]) = pr4;
    __syncthreads();
    float4 rj = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int w = 0; w < 8; ++w) {
        const float4 a = *reinterpret_cast<const float4*>(&sh.red_r[w][4 * ln]);
        rj.x += a.x; rj.y += a.y; rj.z += a.z; rj.w += a.w;
    }
    float4 dv;
    dv.x = __fmul_rn(beta, sh.v[4 * ln + 0] - rj.x);
    dv.y = __fmul_rn(beta, sh.v[4 * ln + 1] - rj.y);
    dv.z = __fmul_rn(beta, sh.v[4 * ln + 2] - rj.z);
    dv.w = __fmul_rn(beta, sh.v[4 * ln + 3] - rj.w);
    float4 po = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int r = 0; r < 16; ++r) {
        const float kh = __fmul_rn(sh.k[warp * 16 + r], kinv);
        const float qh = __fmul_rn(__fmul_rn(sh.q[warp * 16 + r], qinv), q_scale);
        s[r].x = __fadd_rn(s[r].x, __fmul_rn(kh, dv.x));
        s[r].y = __fadd_rn(s[r].y, __fmul_rn(kh, dv.y));
        s[r].z = __fadd_rn(s[r].z, __fmul_rn(kh, dv.z));
        s[r].w = __fadd_rn(s[r].w, __fmul_rn(kh, dv.w));
        po.x += s[r].x * qh; po.y += s[r].y * qh; po.z += s[r].z * qh; po.w += s[r].w * qh;
    }
    *reinterpret_cast<float4*>(&sh.red_o[warp][4 * ln]) = po;
    {
        float4* So = reinterpret_cast<float4*>(S_tile);
#pragma unroll
        for (int r = 0; r < 16; ++r) So[(warp * 16 + r) * 32 + ln] = s[r];
    }
    __syncthreads();
    float o = 0.f;
    if (tid < 128) {
#pragma unroll
        for (int w = 0; w < 8; ++w) o += sh.red_o[w][tid];
        const float oo = warp_sum(o * o);
        if (ln == 0) sh.osum[warp] = oo;
    }
    __syncthreads();
    if (tid < 128) {
        const float ms = (sh.osum[0] + sh.osum[1] + sh.osum[2] + sh.osum[3]) * (1.0f / 128.0f);
        float n = __fmul_rn(o, rsqrt_acc(ms + kEps));
        n = __fmul_rn(nw_in, n);
        const float z = z_in;
        y_row[h * 128 + tid] = f2bf(__fmul_rn(n, silu_acc(z)));
#pragma unroll
        for (int kind = 0; kind < 3; ++kind)
#pragma unroll
            for (int j = 0; j < 3; ++j) win[j * kConvCh + ch[kind]] = f2bf(wnew[kind][j]);
    }
    __syncthreads();
}

// ---- attention: one (lane, kv head, page) unit by the whole CTA -----------------------------------
// Partial record per (lane, head, page): [0] = max score m, [1] = sum exp(s - m), [4..259] = sum
// exp(s - m) V.  The unit that owns the page of the new position appends k (norm + rope, bf16) and v.
constexpr int kPartStride = 260;

__device__ __forceinline__ void attn_unit(float* scratch, const uint16_t* __restrict__ pr, const SmallLayer& L,
                                          const SmallStepParams& p, int lane_id, int kvh, int pg, int n_ctx) {
    constexpr int kOffK = 4096, kOffV = 4608;
    const int tid = threadIdx.x, warp = tid >> 5, ln = tid & 31;
    float* q_s = scratch;                  // [4][256]
    float* sc = q_s + 4 * kHeadDim;        // [4][64]
    float* part = sc + 4 * kKvPage;        // [8][4][256]
    const int slot = n_ctx - 1;
    const int* table = p.table + ((size_t)lane_id * kAttnLayers + L.slot) * p.pages_per_lane;
    const size_t page_base = (size_t)table[pg] * kPageElems + (size_t)kvh * kKvPage * kHeadDim;
    const int p0 = pg * kKvPage;
    const int count = (n_ctx - p0) < kKvPage ? (n_ctx - p0) : kKvPage;

    if (warp < 4) {
        const int head = kvh * 4 + warp;
        float x[8];
        unpack8(__ldcg(reinterpret_cast<const uint4*>(pr + head * 2 * kHeadDim + 8 * ln)), x);
        head_norm_rope(x, L.q_norm, ln, slot, p.inv_freq);
#pragma unroll
        for (int e = 0; e < 8; ++e) q_s[warp * kHeadDim + 8 * ln + e] = x[e];
    } else if (slot >= p0 && slot < p0 + kKvPage) {
        if (warp == 4) {
            float x[8];
            unpack8(__ldcg(reinterpret_cast<const uint4*>(pr + kOffK + kvh * kHeadDim + 8 * ln)), x);
            head_norm_rope(x, L.k_norm, ln, slot, p.inv_freq);
            *reinterpret_cast<uint4*>(p.kpool + page_base + (size_t)(slot - p0) * kHeadDim + 8 * ln) = pack8(x);
        } else if (warp == 5) {
            *reinterpret_cast<uint4*>(p.vpool + page_base + (size_t)(slot - p0) * kHeadDim + 8 * ln) =
                __ldcg(reinterpret_cast<const uint4*>(pr + kOffV + kvh * kHeadDim + 8 * ln));
        }
    }
    __syncthreads();

    // scores of this page: warp w takes positions 8w .. 8w+7
    {
        float qr[4][8];
#pragma unroll
        for (int hh = 0; hh < 4; ++hh)
#pragma unroll
            for (int e = 0; e < 8; ++e) qr[hh][e] = q_s[hh * kHeadDim + 8 * ln + e];
        uint4 kv[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const int j = warp * 8 + u;
            kv[u] = j < count ? *reinterpret_cast<const uint4*>(p.kpool + page_base + (size_t)j * kHeadDim + 8 * ln)
                              : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            float kf[8];
            unpack8(kv[u], kf);
            float d[4];
#pragma unroll
            for (int hh = 0; hh < 4; ++hh) {
                float a = 0.f;
#pragma unroll
                for (int e = 0; e < 8; ++e) a += qr[hh][e] * kf[e];
                d[hh] = warp_sum(a);
            }
            const int j = warp * 8 + u;
            if (ln < 4) {
                const float v = ln == 0 ? d[0] : (ln == 1 ? d[1] : (ln == 2 ? d[2] : d[3]));
                sc[ln * kKvPage + j] = j < count ? v * 0.0625f : -INFINITY;
            }
        }
    }
    __syncthreads();
    // per-head statistics of the page; sc <- exp(s - m)
    if (warp < 4) {
        float* s = sc + warp * kKvPage;
        const float a = s[ln], b = s[ln + 32];
        const float m = warp_max(fmaxf(a, b));
        const float ea = expf(a - m), eb = expf(b - m);
        s[ln] = ea; s[ln + 32] = eb;
        const float l = warp_sum(ea + eb);
        if (ln == 0) {
            float* rec = p.attn_part + (((size_t)lane_id * kQHeads + kvh * 4 + warp) * p.pages_per_lane + pg) * kPartStride;
            rec[0] = m; rec[1] = l;
        }
    }
    __syncthreads();
    // partial P.V: warp w takes positions 8w .. 8w+7, a lane holds 8 dims
    {
        float acc[4][8];
#pragma unroll
        for (int hh = 0; hh < 4; ++hh)
#pragma unroll
            for (int e = 0; e < 8; ++e) acc[hh][e] = 0.f;
        uint4 vv[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const int j = warp * 8 + u;
            vv[u] = j < count ? *reinterpret_cast<const uint4*>(p.vpool + page_base + (size_t)j * kHeadDim + 8 * ln)
                              : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const int j = warp * 8 + u;
            if (j >= count) break;
            float vf[8];
            unpack8(vv[u], vf);
#pragma unroll
            for (int hh = 0; hh < 4; ++hh) {
                const float wgt = sc[hh * kKvPage + j];
#pragma unroll
                for (int e = 0; e < 8; ++e) acc[hh][e] += wgt * vf[e];
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
    for (int idx = tid; idx < 4 * kHeadDim; idx += kThreads) {
        const int hh = idx >> 8, dd = idx & 255;
        float a = 0.f;
#pragma unroll
        for (int w = 0; w < 8; ++w) a += part[(w * 4 + hh) * kHeadDim + dd];
        p.attn_part[(((size_t)lane_id * kQHeads + kvh * 4 + hh) * p.pages_per_lane + pg) * kPartStride + 4 + dd] = a;
    }
    __syncthreads();
}

// merge the page partials of one (lane, head): out = sum_u e^(m_u - M) acc_u / sum_u e^(m_u - M) l_u,
// rounded to bf16, times the bf16 sigmoid gate.  One CTA, thread = output dim.
__device__ __forceinline__ void attn_combine(const SmallStepParams& p, const uint16_t* __restrict__ pr, int lane_id,
                                             int head, int P) {
    const int d = threadIdx.x;
    const float* rec0 = p.attn_part + ((size_t)lane_id * kQHeads + head) * p.pages_per_lane * kPartStride;
    float M = -INFINITY;
    for (int u = 0; u < P; ++u) M = fmaxf(M, __ldcg(rec0 + (size_t)u * kPartStride));
    float Lsum = 0.f, acc = 0.f;
    for (int u = 0; u < P; ++u) {
        const float* rec = rec0 + (size_t)u * kPartStride;
        const float w = expf(__ldcg(rec) - M);
        Lsum += w * __ldcg(rec + 1);
        acc += w * __ldcg(rec + 4 + d);
    }
    const float a = bfround(__fdiv_rn(acc, Lsum));
    const float gate = ldcg_bf(pr + head * 2 * kHeadDim + kHeadDim + d);
    p.mix[(size_t)lane_id * (kQHeads * kHeadDim) + head * kHeadDim + d] = f2bf(a * bfround(sigmoid_acc(gate)));
}

// ---- L2 prefetch of the weight rows this CTA will use in weight phase `wp` ----------------------
// wp = 4 * layer + kind (0 in-proj, 1 out-proj, 2 gate/up, 3 down); wp = 96 is the head's first rounds.
__device__ __forceinline__ void prefetch_weight_phase(const SmallStepParams& p, int wp) {
    const int G = gridDim.x, cta = blockIdx.x;
    const int warp = threadIdx.x >> 5, ln = threadIdx.x & 31;
    if (ln != 0 || wp > 4 * kLayers) return;
    if (wp == 4 * kLayers) {
        const int ngroups = p.vocab / 8;
        for (int r = 0; r < 2; ++r) {
            const int gidx = (r * 8 + warp) * G + cta;
            if (gidx < ngroups) l2_prefetch(p.embed + (size_t)gidx * 8 * kHidden, 8 * kHidden * 2);
        }
        return;
    }
    const SmallLayer& L = p.layers[wp >> 2];
    const int kind = wp & 3;
    if (kind == 0 || kind == 2) {
        const uint16_t* W = kind == 0 ? L.in_w : L.gu_w;
        const int ngroups = (kind == 0 ? L.in_n : 2 * kFF) / 8;
        for (int gidx = warp * G + cta; gidx < ngroups; gidx += 8 * G)
            l2_prefetch(W + (size_t)gidx * 8 * kHidden, 8 * kHidden * 2);
    } else if (warp == 0 && cta < kHidden / 8) {
        const int K = kind == 1 ? 2048 : kFF;
        l2_prefetch((kind == 1 ? L.out_w : L.down_w) + (size_t)cta * 8 * K, 8 * K * 2);
    }
}

__global__ void __launch_bounds__(kThreads, 1) small_step_kernel(SmallStepParams p) {
    extern __shared__ __align__(16) unsigned char dyn_smem[];
    uint16_t* xs = reinterpret_cast<uint16_t*>(dyn_smem);
    __shared__ GdnShared gsh;
    __shared__ __align__(16) float red[8 * 128];
    __shared__ ArgMax hbest[8][16];
    __shared__ int abort_s;

    const int G = gridDim.x, cta = blockIdx.x, M = p.lanes;
    const int tid = threadIdx.x, warp = tid >> 5, ln = tid & 31, g = ln >> 2, t = ln & 3;
    if (p.status != nullptr && *p.status != 0) return;
    if (tid == 0) abort_s = 0;
    __syncthreads();
    unsigned phase = 0;
#define GRID_BARRIER()                                                          \
    do {                                                                        \
        if (p.trace != nullptr && cta == 0 && tid == 0) p.trace[2 * phase + 1] = global_ns(); \
        ++phase;                                                                \
        if (!grid_barrier(p.bar, phase * (unsigned)G, p.status, &abort_s)) return; \
        if (p.trace != nullptr && cta == 0 && tid == 0) p.trace[2 * phase] = global_ns(); \
    } while (0)
    if (p.trace != nullptr && cta == 0 && tid == 0) p.trace[0] = global_ns();

    prefetch_weight_phase(p, 0);
    prefetch_weight_phase(p, 1);
    int cur = 0;
    const int cap = p.pages_per_lane * kKvPage;
    const int my_group = warp * G + cta;          // this warp's 8-row group in the warp-per-group phases
    const bool has_unit = cta < kHidden / 8;      // this CTA's 8-row unit in the K-split phases
    uint4 wa[16], wb[16];                         // weight registers of the NEXT projection phase
    wg_load_half(wa, p.layers[0].in_w, my_group * 8, p.layers[0].in_n, 0);

    for (int l = 0; l < kLayers; ++l) {
        const SmallLayer& L = p.layers[l];
        uint16_t* resid_cur = p.resid + (size_t)cur * 16 * kHidden;
        uint16_t* resid_nxt = p.resid + (size_t)(cur ^ 1) * 16 * kHidden;

        // ================= in-projection (x = norm of the running residual) =========================
        {
            const int N = L.in_n, ngroups = N / 8;
            const bool mine = my_group < ngroups;
            if (mine) wg_load_half(wb, L.in_w, my_group * 8, N, 1);
            prefetch_weight_phase(p, 4 * l + 2);
            if (tid == 32) {                    // state this CTA's mixer items will touch
                if (!L.attn) {
                    for (int item = cta; item < M * kGdnHeads; item += G)
                        l2_prefetch(p.S + ((size_t)L.slot * M * kGdnHeads + item) * (kDk * kDv), kDk * kDv * 4);
                } else {
                    const int per_lane = kKvHeads * p.pages_per_lane;
                    for (int u = cta; u < M * per_lane; u += G) {
                        const int lane_id = u / per_lane, rem = u % per_lane;
                        const int kvh = rem / p.pages_per_lane, pg = rem % p.pages_per_lane;
                        int n_ctx = p.pos[lane_id] + 1;
                        n_ctx = n_ctx < cap ? n_ctx : cap;
                        if (pg * kKvPage >= n_ctx) continue;
                        const int* table = p.table + ((size_t)lane_id * kAttnLayers + L.slot) * p.pages_per_lane;
                        const size_t off = (size_t)table[pg] * kPageElems + (size_t)kvh * kKvPage * kHeadDim;
                        l2_prefetch(p.kpool + off, kKvPage * kHeadDim * 2);
                        l2_prefetch(p.vpool + off, kKvPage * kHeadDim * 2);
                    }
                }
            }
            if (l == 0) {
                norm_rows_to_smem(xs, nullptr, p.in_tok, p.embed, p.vocab, nullptr, L.input_norm, M,
                                  cta == 0 ? resid_cur : nullptr, nullptr);
            } else {
                norm_rows_to_smem(xs, resid_cur, nullptr, nullptr, 0, p.delta, L.input_norm, M,
                                  cta == 0 ? resid_nxt : nullptr, nullptr);
                cur ^= 1;
            }
            __syncthreads();
            if (mine) {
                float acc[4];
                wg_compute(xs, wa, wb, acc);
                const int col = my_group * 8 + 2 * t;
                if (g < M) *reinterpret_cast<uint32_t*>(p.proj + (size_t)g * N + col) = pack_bf2(acc[0], acc[1]);
                if (g + 8 < M) *reinterpret_cast<uint32_t*>(p.proj + (size_t)(g + 8) * N + col) = pack_bf2(acc[2], acc[3]);
            }
        }
        GRID_BARRIER();

        // ================= mixer ====================================================================
        prefetch_weight_phase(p, 4 * l + 3);
        if (!L.attn) {
            for (int item = cta; item < M * kGdnHeads; item += G) {
                const int lane_id = item / kGdnHeads, h = item % kGdnHeads;
                gdn_item(gsh, p.proj + (size_t)lane_id * kGdnProjN, L.conv_w, L.A_log, L.dt_bias, L.gdn_norm,
                         p.S + (((size_t)L.slot * M + lane_id) * kGdnHeads + h) * (kDk * kDv),
                         p.win + ((size_t)L.slot * M + lane_id) * 3 * kConvCh, h, p.mix + (size_t)lane_id * kValueDim);
            }
        } else {
            const int per_lane = kKvHeads * p.pages_per_lane;
            for (int u = cta; u < M * per_lane; u += G) {
                const int lane_id = u / per_lane, rem = u % per_lane;
                const int kvh = rem / p.pages_per_lane, pg = rem % p.pages_per_lane;
                int n_ctx = p.pos[lane_id] + 1;
                n_ctx = n_ctx < cap ? n_ctx : cap;
                if (pg * kKvPage >= n_ctx) continue;
                attn_unit(reinterpret_cast<float*>(dyn_smem), p.proj + (size_t)lane_id * kAttnProjN, L, p, lane_id, kvh, pg, n_ctx);
            }
            GRID_BARRIER();
            for (int item = cta; item < M * kQHeads; item += G) {
                const int lane_id = item / kQHeads, head = item % kQHeads;
                int n_ctx = p.pos[lane_id] + 1;
                n_ctx = n_ctx < cap ? n_ctx : cap;
                attn_combine(p, p.proj + (size_t)lane_id * kAttnProjN, lane_id, head, (n_ctx + kKvPage - 1) / kKvPage);
            }
        }
        if (has_unit) cu_load<2048>(wa, L.out_w, cta * 8, kHidden);
        GRID_BARRIER();

        // ================= out-projection ===========================================================
        prefetch_weight_phase(p, 4 * l + 4);
        rows_to_smem(xs, XLD2, p.mix, 2048, M);
        __syncthreads();
        if (has_unit) cu_compute<2048, XLD2>(xs, wa, cta * 8, kHidden, M, red, p.delta);
        const bool gu_mine = my_group < 2 * kFF / 8;
        if (gu_mine) wg_load_half(wa, L.gu_w, my_group * 8, 2 * kFF, 0);
        GRID_BARRIER();

        // ================= gate / up with SwiGLU (x = norm of residual + mixer delta) ===============
        if (gu_mine) wg_load_half(wb, L.gu_w, my_group * 8, 2 * kFF, 1);
        prefetch_weight_phase(p, 4 * l + 5);
        resid_cur = p.resid + (size_t)cur * 16 * kHidden;
        resid_nxt = p.resid + (size_t)(cur ^ 1) * 16 * kHidden;
        norm_rows_to_smem(xs, resid_cur, nullptr, nullptr, 0, p.delta, L.post_norm, M, cta == 0 ? resid_nxt : nullptr, nullptr);
        cur ^= 1;
        __syncthreads();
        if (gu_mine) {
            float acc[4];
            wg_compute(xs, wa, wb, acc);
            const int f = my_group * 4 + t;
            if (g < M) p.act[(size_t)g * kFF + f] = swiglu_bf16(acc[0], acc[1]);
            if (g + 8 < M) p.act[(size_t)(g + 8) * kFF + f] = swiglu_bf16(acc[2], acc[3]);
        }
        if (has_unit) cu_load<kFF>(wa, L.down_w, cta * 8, kHidden);
        GRID_BARRIER();

        // ================= down-projection ==========================================================
        prefetch_weight_phase(p, 4 * l + 6);
        rows_to_smem(xs, XLD3, p.act, kFF, M);
        __syncthreads();
        if (has_unit) cu_compute<kFF, XLD3>(xs, wa, cta * 8, kHidden, M, red, p.delta);
        if (l + 1 < kLayers) {
            if (my_group < p.layers[l + 1].in_n / 8) wg_load_half(wa, p.layers[l + 1].in_w, my_group * 8, p.layers[l + 1].in_n, 0);
        } else if (my_group < p.vocab / 8) {
            wg_load_half(wa, p.embed, my_group * 8, p.vocab, 0);
        }
        GRID_BARRIER();
    }

    // ================= tied head + argmax ===========================================================
    {
        const int ngroups = p.vocab / 8;
        if (my_group < ngroups) wg_load_half(wb, p.embed, my_group * 8, p.vocab, 1);
        norm_rows_to_smem(xs, p.resid + (size_t)cur * 16 * kHidden, nullptr, nullptr, 0, p.delta, p.final_norm, M, nullptr,
                          cta == 0 ? p.normed : nullptr);
        __syncthreads();
        float bv0 = -INFINITY, bv1 = -INFINITY;
        int bi0 = 0x7fffffff, bi1 = 0x7fffffff;
        for (int gidx = my_group; gidx < ngroups; gidx += 8 * G) {
            const int ahead = gidx + 16 * G;
            if (ln == 0 && ahead < ngroups) l2_prefetch(p.embed + (size_t)ahead * 8 * kHidden, 8 * kHidden * 2);
            float acc[4];
            wg_compute(xs, wa, wb, acc);
            const int nxt = gidx + 8 * G;               // next round's weights fly under this round's argmax
            if (nxt < ngroups) {
                wg_load_half(wa, p.embed, nxt * 8, p.vocab, 0);
                wg_load_half(wb, p.embed, nxt * 8, p.vocab, 1);
            }
            const int col = gidx * 8 + 2 * t;
            if (better(acc[0], col, bv0, bi0)) { bv0 = acc[0]; bi0 = col; }
            if (better(acc[1], col + 1, bv0, bi0)) { bv0 = acc[1]; bi0 = col + 1; }
            if (better(acc[2], col, bv1, bi1)) { bv1 = acc[2]; bi1 = col; }
            if (better(acc[3], col + 1, bv1, bi1)) { bv1 = acc[3]; bi1 = col + 1; }
        }
#pragma unroll
        for (int o = 1; o <= 2; o <<= 1) {
            const float ov0 = __shfl_xor_sync(0xffffffffu, bv0, o), ov1 = __shfl_xor_sync(0xffffffffu, bv1, o);
            const int oi0 = __shfl_xor_sync(0xffffffffu, bi0, o), oi1 = __shfl_xor_sync(0xffffffffu, bi1, o);
            if (better(ov0, oi0, bv0, bi0)) { bv0 = ov0; bi0 = oi0; }
            if (better(ov1, oi1, bv1, bi1)) { bv1 = ov1; bi1 = oi1; }
        }
        if (t == 0) { hbest[warp][g] = ArgMax{bv0, bi0}; hbest[warp][g + 8] = ArgMax{bv1, bi1}; }
        __syncthreads();
        if (tid < 16) {
            ArgMax b = hbest[0][tid];
#pragma unroll
            for (int w = 1; w < 8; ++w)
                if (better(hbest[w][tid].v, hbest[w][tid].i, b.v, b.i)) b = hbest[w][tid];
            p.head_part[(size_t)cta * 16 + tid] = b;
        }
    }
    GRID_BARRIER();
    if (cta == 0) {
        for (int row = warp; row < M; row += 8) {
            float bv = -INFINITY;
            int bi = 0x7fffffff;
            for (int c = ln; c < G; c += 32) {
                const float v = __ldcg(&p.head_part[(size_t)c * 16 + row].v);
                const int i = __ldcg(&p.head_part[(size_t)c * 16 + row].i);
                if (better(v, i, bv, bi)) { bv = v; bi = i; }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
                const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
                if (better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
            }
            if (ln == 0) { p.out_tok[row] = bi; p.pos[row] += 1; }
        }
    }
#undef GRID_BARRIER
}

}  // namespace

cudaError_t launch_small_step(const SmallStepParams& p, cudaStream_t st) {
    if (p.lanes < 1 || p.lanes > kSmallStepMaxLanes || (p.vocab & 7)) return cudaErrorInvalidValue;
    static int grid = 0;
    if (grid == 0) {
        int dev = 0, sms = 0;
        cudaError_t e = cudaGetDevice(&dev);
        if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        if (e == cudaSuccess)
            e = cudaFuncSetAttribute(small_step_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmallSmem);
        if (e != cudaSuccess) return e;
        int per_sm = 0;
        e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, small_step_kernel, kThreads, kSmallSmem);
        if (e != cudaSuccess) return e;
        if (per_sm < 1) return cudaErrorLaunchOutOfResources;
        grid = sms;                       // one CTA per SM: all co-resident, which the grid barrier needs
    }
    cudaError_t e = cudaMemsetAsync(p.bar, 0, sizeof(unsigned), st);
    if (e != cudaSuccess) return e;
    // cooperative launch: the runtime refuses the launch unless every CTA can be resident at once
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = kSmallSmem;
    cfg.stream = st;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeCooperative;
    at[0].val.cooperative = 1;
    cfg.attrs = at;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, small_step_kernel, p);
}

}  // namespace q35
