// Chunked (chunk = 64 tokens) GatedDeltaNet prefill: the UT-transform form of the delta rule.
//
// For a body that carries T >= 32 tokens per lane the token-by-token recurrence is replaced by
//   (1) gdn_conv_prep_kernel : causal conv1d + SiLU over all T rows of a lane, in place over the
//       raw q|k|v columns of the projection buffer, and the conv-window roll (SiLU of a bf16 value
//       by table: the pass is otherwise bound by instruction issue, not by memory);
//   (2) gdn_chunk_tc_kernel  : one CTA per (head, lane) walks the chunks with the 128x128 f32 state
//       resident in shared memory.  Per chunk: row scalars (L2 norms, beta, log-decay prefix sum),
//       G = K K^T and P = Q K^T masked by the pairwise decay, q S and k S in one pass over the state,
//       ONE unit-lower-triangular solve
//           v_new = inv(I + L) (beta v - beta e^cum k_hat S),
//           o = (e^cum q) S + intra v_new ;  S = e^cumC S + (e^(cumC-cum) k)^T v_new
//       and the gated RMSNorm of o: the algebra of the reference's chunked form
//       (speccheck/specimpl.py:187-235), every product on the tensor pipe with f32-grade operands
//       (see the kernel's comment).  Rows past T are padded with beta = 0, g = 0, q = k = v = 0
//       (they neither read nor write S).
//   (2') gdn_chunk_umma_kernel : the same scan with its two 128-wide products (state read-out and state
//       update) on tcgen05 with tensor-memory accumulators - the default; (2) stays as the cross-check
//       (Q35_GDN_CHUNK=mma).
// The reference engine ships only the sequential span kernel (engine/gdn_rec_reg16_kernels.h); its
// chunked prototype is disabled (engine/kernels_gdn.cpp:430-446).
#include <cstdlib>

#include "q35_common.cuh"
#include "q35_async.cuh"
#include "q35_tcgen05.cuh"

namespace q35 {

namespace {

constexpr int C = 64;                  // chunk length
constexpr int KQ_LD = 136;             // bf16 row stride of the q / k chunk tiles (272 B: conflict-free 16-B reads)
constexpr int T_LD = 68;               // f32 row stride of the 64x64 matrices
constexpr int kOffZ = 6144, kOffB = 8192, kOffA = 8208;


// SiLU of a bf16 value rounded to bf16 is a function of 16 bits: the conv pass, which is bound by
// instruction issue (an accurate exp and an IEEE divide per element), looks it up instead.  The
// table is filled on the device by the same expression the step kernel evaluates, so both agree bit
// for bit; 128 KiB, hot lines stay in L1.
__device__ uint16_t g_silu_bf16[65536];
__global__ void silu_table_kernel() {
    const int b = blockIdx.x * blockDim.x + threadIdx.x;
    g_silu_bf16[b] = f2bf(silu_acc(bf2f((uint16_t)b)));
}

// ---- (1) conv + SiLU over a lane's T rows, in place; window roll -------------------------------
// grid (lanes, 6), 128 threads, 8 adjacent channels per thread (16-byte loads, eight rows in flight).
__global__ void __launch_bounds__(128)
gdn_conv_prep_kernel(uint16_t* __restrict__ proj, const uint16_t* __restrict__ conv_w,
                     uint16_t* __restrict__ win0, uint16_t* __restrict__ win1, uint16_t* __restrict__ win2,
                     const int* __restrict__ sel, int T) {
    const int lane_id = blockIdx.x;
    const int c = (blockIdx.y * 128 + threadIdx.x) * 8;
    const int live = sel != nullptr ? sel[lane_id] : 0;
    uint16_t* win = (live == 0 ? win0 : (live == 1 ? win1 : win2)) + (size_t)lane_id * 3 * kConvCh;
    float tap[8][4], w[8][3];
#pragma unroll
    for (int q = 0; q < 4; ++q) {            // taps of channels 2q, 2q + 1
        const uint4 tw = *reinterpret_cast<const uint4*>(conv_w + (size_t)(c + 2 * q) * 4);
        tap[2 * q][0] = lo_bf(tw.x); tap[2 * q][1] = hi_bf(tw.x); tap[2 * q][2] = lo_bf(tw.y); tap[2 * q][3] = hi_bf(tw.y);
        tap[2 * q + 1][0] = lo_bf(tw.z); tap[2 * q + 1][1] = hi_bf(tw.z); tap[2 * q + 1][2] = lo_bf(tw.w); tap[2 * q + 1][3] = hi_bf(tw.w);
    }
#pragma unroll
    for (int j = 0; j < 3; ++j) {
        const uint4 v = *reinterpret_cast<const uint4*>(win + j * kConvCh + c);
        const uint32_t vw[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int q = 0; q < 4; ++q) { w[2 * q][j] = lo_bf(vw[q]); w[2 * q + 1][j] = hi_bf(vw[q]); }
    }
    uint16_t* p = proj + (size_t)lane_id * T * kGdnProjN + c;
    for (int t0 = 0; t0 < T; t0 += 8) {
        uint4 rv[8];
#pragma unroll
        for (int u = 0; u < 8; ++u)
            if (t0 + u < T) rv[u] = *reinterpret_cast<const uint4*>(p + (size_t)(t0 + u) * kGdnProjN);
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            if (t0 + u < T) {
                const uint32_t rw[4] = {rv[u].x, rv[u].y, rv[u].z, rv[u].w};
                uint32_t ow[4];
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    float o2[2];
#pragma unroll
                    for (int e2 = 0; e2 < 2; ++e2) {
                        const int e = 2 * q + e2;
                        const float raw = e2 == 0 ? lo_bf(rw[q]) : hi_bf(rw[q]);
                        float acc = __fmul_rn(w[e][0], tap[e][0]);
                        acc = __fadd_rn(acc, __fmul_rn(w[e][1], tap[e][1]));
                        acc = __fadd_rn(acc, __fmul_rn(w[e][2], tap[e][2]));
                        acc = __fadd_rn(acc, __fmul_rn(raw, tap[e][3]));
                        o2[e2] = bf2f(g_silu_bf16[f2bf(acc)]);             // = bfround(silu(bfround(acc)))
                        w[e][0] = w[e][1]; w[e][1] = w[e][2]; w[e][2] = raw;
                    }
                    ow[q] = pack_bf2(o2[0], o2[1]);
                }
                *reinterpret_cast<uint4*>(p + (size_t)(t0 + u) * kGdnProjN) = make_uint4(ow[0], ow[1], ow[2], ow[3]);
            }
        }
    }
#pragma unroll
    for (int j = 0; j < 3; ++j) {
        uint32_t ow[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) ow[q] = pack_bf2(w[2 * q][j], w[2 * q + 1][j]);
        *reinterpret_cast<uint4*>(win + j * kConvCh + c) = make_uint4(ow[0], ow[1], ow[2], ow[3]);
    }
}

__device__ __forceinline__ void unpack8f(const uint4& v, float (&f)[8]) {
    f[0] = lo_bf(v.x); f[1] = hi_bf(v.x); f[2] = lo_bf(v.y); f[3] = hi_bf(v.y);
    f[4] = lo_bf(v.z); f[5] = hi_bf(v.z); f[6] = lo_bf(v.w); f[7] = hi_bf(v.w);
}

// ---- (2') the chunk scan on the tensor pipe ------------------------------------------------------
// Every product runs as warp-level mma: G and P from the bf16 tiles (m16n8k16, exact products), the
// f32 products as split-TF32 (m16n8k8): an f32 operand x is fed as hi = x with the low 13 mantissa
// bits cleared and lo = x - hi, and a.b ~ a_lo b_hi + a_hi b_lo + a_hi b_hi (relative error ~2^-20
// per product); q and k are bf16 values, exact as TF32, so their products need two instructions.
// Order of a chunk (warp = 16 rows x 64 columns of a 64 x 128 result unless said otherwise):
//   loads (q, k by cp.async, v and gate inputs to registers; on the first chunk the 64 KiB state by
//   cp.async behind them) -> row scalars -> beta v -> G, P -> [state landed] inverses of the four
//   16 x 16 diagonal blocks of I + L (64 threads, forward substitution) -> q S and k S in one pass
//   over the state -> right-hand side beta v - (beta e^cum / |k|) (k S) -> blocked solve, a warp
//   walking the four block rows of its own 16 columns, X_b = inv(D_b) (B_b - sum_{c<b} L_bc X_c) ->
//   intra v_new, output scaling, gated RMSNorm, y -> state update (warp = 16 rows of S).
// Forming the right-hand side before the solve halves the solve and drops one 64 x 128 x 128
// product against  inv(I + L) (beta e^cum k_hat).  Row strides make fragment loads conflict-free
// (A-type rows: stride = 4 mod 32 words, B-type rows: stride = 8 mod 32 words).  Work that grows
// with the row tile (G / P blocks, intra columns) is dealt so that the two warps of a scheduler
// get tiles mt and 3 - mt.
constexpr int S_LD = 136;              // f32 row stride of the state (B operand)
constexpr int V_LD = 136;              // f32 row stride of the right-hand side / v_new (B operand)
constexpr size_t kChunkTcSmem = (size_t)128 * S_LD * 4 + (size_t)C * V_LD * 4 +
                                2 * (size_t)C * KQ_LD * 2 + 3 * (size_t)C * T_LD * 4 + 8 * C * 4 + 2 * C * 4;

__device__ __forceinline__ void ldsm4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_tf32(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm(
        "mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// x = hi + lo exactly; hi carries the top 11 significand bits, lo the rest (the pipe reads its top 11)
__device__ __forceinline__ void split_tf32(float x, uint32_t& hi, uint32_t& lo) {
    hi = __float_as_uint(x) & 0xffffe000u;
    lo = __float_as_uint(__fsub_rn(x, __uint_as_float(hi)));
}

// Split-TF32 products of one A fragment against NT B tiles (b0 = B[k0 + t][n], b1 = B[k0 + t + 4][n], tiles
// 8 columns apart, optional row scales), pass by pass so that no two consecutive instructions share an accumulator.
template <int NT, bool A_EXACT>
__device__ __forceinline__ void mma_row(float (&acc)[NT][4], const uint32_t (&ahi)[4], const uint32_t (&alo)[4],
                                        const float* __restrict__ b_row0, const float* __restrict__ b_row1,
                                        float w0, float w1) {
    uint32_t bh[NT][2], bl[NT][2];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        split_tf32(b_row0[8 * nt] * w0, bh[nt][0], bl[nt][0]);
        split_tf32(b_row1[8 * nt] * w1, bh[nt][1], bl[nt][1]);
    }
    if (!A_EXACT) {
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) mma_tf32(acc[nt], alo, bh[nt][0], bh[nt][1]);
    }
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) mma_tf32(acc[nt], ahi, bl[nt][0], bl[nt][1]);
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) mma_tf32(acc[nt], ahi, bh[nt][0], bh[nt][1]);
}

// Two exact (bf16-valued) A fragments against the same NT B tiles: the split of B is shared.
template <int NT>
__device__ __forceinline__ void mma_row_pair(float (&acc0)[NT][4], float (&acc1)[NT][4], const uint32_t (&a0)[4],
                                             const uint32_t (&a1)[4], const float* __restrict__ b_row0,
                                             const float* __restrict__ b_row1) {
    uint32_t bh[NT][2], bl[NT][2];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        split_tf32(b_row0[8 * nt], bh[nt][0], bl[nt][0]);
        split_tf32(b_row1[8 * nt], bh[nt][1], bl[nt][1]);
    }
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) { mma_tf32(acc0[nt], a0, bl[nt][0], bl[nt][1]); mma_tf32(acc1[nt], a1, bl[nt][0], bl[nt][1]); }
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) { mma_tf32(acc0[nt], a0, bh[nt][0], bh[nt][1]); mma_tf32(acc1[nt], a1, bh[nt][0], bh[nt][1]); }
}

// The same with one accumulator set per pass (summed by the caller): three times the independent
// chains, for the short dependent products of the blocked solve.
template <int NT>
__device__ __forceinline__ void mma_row3(float (&acc_hh)[NT][4], float (&acc_lh)[NT][4], float (&acc_hl)[NT][4],
                                         const uint32_t (&ahi)[4], const uint32_t (&alo)[4],
                                         const float* __restrict__ b_row0, const float* __restrict__ b_row1) {
    uint32_t bh[NT][2], bl[NT][2];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        split_tf32(b_row0[8 * nt], bh[nt][0], bl[nt][0]);
        split_tf32(b_row1[8 * nt], bh[nt][1], bl[nt][1]);
    }
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        mma_tf32(acc_lh[nt], alo, bh[nt][0], bh[nt][1]);
        mma_tf32(acc_hl[nt], ahi, bl[nt][0], bl[nt][1]);
        mma_tf32(acc_hh[nt], ahi, bh[nt][0], bh[nt][1]);
    }
}

__global__ void __launch_bounds__(256, 1)
gdn_chunk_tc_kernel(const uint16_t* __restrict__ proj, const uint16_t* __restrict__ A_log,
                    const uint16_t* __restrict__ dt_bias, const uint16_t* __restrict__ norm_w,
                    float* __restrict__ S0, float* __restrict__ S1, float* __restrict__ S2,
                    const int* __restrict__ sel, uint16_t* __restrict__ y, int T) {
    extern __shared__ __align__(16) unsigned char smem_chunk[];
    float* S_s = reinterpret_cast<float*>(smem_chunk);                 // [128][136]  S[dk][dv]
    float* V_s = S_s + 128 * S_LD;                                     // [64][136]   beta v, right-hand side, v_new
    uint16_t* K_s = reinterpret_cast<uint16_t*>(V_s + C * V_LD);       // [64][136] bf16
    uint16_t* Q_s = K_s + C * KQ_LD;                                   // [64][136] bf16
    float* Tri_s = reinterpret_cast<float*>(Q_s + C * KQ_LD);          // [64][68]
    float* Int_s = Tri_s + C * T_LD;                                   // [64][68]
    float* Tinv_s = Int_s + C * T_LD;                                  // [64][68]   inverses of the diagonal blocks
    float* sc = Tinv_s + C * T_LD;                                     // 8 x [64] row scalars
    float* red_s = sc + 8 * C;                                         // [2][64] sum of squares per column half
    float* cum_s = sc;
    float* beta_s = sc + 64;
    float* kinv_s = sc + 128;
    float* qsc_s = sc + 192;
    float* ecum_s = sc + 256;
    float* kout_s = sc + 320;
    float* g_s = sc + 384;
    float* qn_s = sc + 448;

    const int h = blockIdx.x, lane_id = blockIdx.y;
    const int tid = threadIdx.x, warp = tid >> 5, ln = tid & 31;
    const int g = ln >> 2, t = ln & 3;                 // fragment coordinates of this lane
    const int live = sel != nullptr ? sel[lane_id] : 0;
    float* S_g = (live == 0 ? S0 : (live == 1 ? S1 : S2)) + ((size_t)lane_id * kGdnHeads + h) * (kDk * kDv);
    const float negA = -expf(bf2f(A_log[h]));
    const float dtb = bf2f(dt_bias[h]);
    const float q_scale = 0.08838834764831845f;

    const int n_chunks = (T + C - 1) / C;
    for (int ck = 0; ck < n_chunks; ++ck) {
        const int t0 = ck * C;
        const int valid = (T - t0) < C ? (T - t0) : C;
        const uint16_t* pr0 = proj + ((size_t)lane_id * T + t0) * kGdnProjN;

        // ---- q, k tiles (bf16, zero rows past T), v pieces and gate inputs: the small requests go out first,
        // the 64 KiB state behind them; it lands while the scalars, G, P and the solve are computed ---------
        for (int i = tid; i < C * 16; i += 256) {
            const int r = i >> 4, cc = i & 15;
            const uint16_t* pr = pr0 + (size_t)(r < valid ? r : 0) * kGdnProjN + h * 128 + cc * 8;
            const uint32_t n = r < valid ? 16u : 0u;                // 0 bytes read = 16 bytes of zeros written
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n"
                         ::"r"(smem_u32(Q_s + r * KQ_LD + cc * 8)), "l"(pr), "r"(n) : "memory");
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n"
                         ::"r"(smem_u32(K_s + r * KQ_LD + cc * 8)), "l"(pr + 2048), "r"(n) : "memory");
        }
        asm volatile("cp.async.commit_group;\n" ::: "memory");
        uint4 vraw[4];                               // this thread's v pieces, used by the right-hand sides
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int i = tid + 256 * u, r = i >> 4, cc = i & 15;
            vraw[u] = make_uint4(0, 0, 0, 0);
            if (r < valid) vraw[u] = *reinterpret_cast<const uint4*>(pr0 + (size_t)r * kGdnProjN + 4096 + h * 128 + cc * 8);
        }
        float b_in = 0.f, a_in = 0.f;
        if (tid < valid) {
            const uint16_t* pr = pr0 + (size_t)tid * kGdnProjN;
            b_in = bf2f(pr[kOffB + h]);
            a_in = bf2f(pr[kOffA + h]);
        }
        if (ck == 0) {
            for (int i = tid; i < 128 * 32; i += 256)
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n"
                             ::"r"(smem_u32(S_s + (i >> 5) * S_LD + (i & 31) * 4)), "l"(S_g + 4 * i) : "memory");
            asm volatile("cp.async.commit_group;\n" ::: "memory");
        }
        if (tid < C) {
            float beta = 0.f, gg = 0.f;
            if (tid < valid) {
                beta = sigmoid_acc(b_in);
                const float sp_in = a_in + dtb;
                const float sp = sp_in > 20.0f ? sp_in : log1pf(expf(sp_in));
                gg = __fmul_rn(negA, sp);
            }
            beta_s[tid] = beta;
            g_s[tid] = gg;
        }
        if (ck == 0) asm volatile("cp.async.wait_group 1;\n" ::: "memory");     // the q, k tiles; the state may still fly
        else asm volatile("cp.async.wait_group 0;\n" ::: "memory");
        __syncthreads();

        // ---- row scalars: L2 norms (warp w takes rows 8w..8w+7), prefix sum of g -----------------
        float my_qs = 0.f, my_ks = 0.f;              // lane rr keeps the sums of row 8 warp + rr
#pragma unroll
        for (int rr = 0; rr < 8; ++rr) {
            const int r = warp * 8 + rr;
            const uint2 kv = *reinterpret_cast<const uint2*>(K_s + r * KQ_LD + ln * 4);
            const uint2 qv = *reinterpret_cast<const uint2*>(Q_s + r * KQ_LD + ln * 4);
            float ks = lo_bf(kv.x) * lo_bf(kv.x) + hi_bf(kv.x) * hi_bf(kv.x) + lo_bf(kv.y) * lo_bf(kv.y) + hi_bf(kv.y) * hi_bf(kv.y);
            float qs = lo_bf(qv.x) * lo_bf(qv.x) + hi_bf(qv.x) * hi_bf(qv.x) + lo_bf(qv.y) * lo_bf(qv.y) + hi_bf(qv.y) * hi_bf(qv.y);
            ks = warp_sum(ks);
            qs = warp_sum(qs);
            if (ln == rr) { my_ks = ks; my_qs = qs; }
        }
        float my_qinv = 0.f;
        if (ln < 8) {
            my_qinv = rsqrt_acc(my_qs + 1e-6f);
            kinv_s[warp * 8 + ln] = rsqrt_acc(my_ks + 1e-6f);
        }
        if (tid == 0) {                      // sequential like the reference's cumsum, but from registers
            float gv[C];
#pragma unroll
            for (int i4 = 0; i4 < C / 4; ++i4) {
                const float4 v = reinterpret_cast<const float4*>(g_s)[i4];
                gv[4 * i4] = v.x; gv[4 * i4 + 1] = v.y; gv[4 * i4 + 2] = v.z; gv[4 * i4 + 3] = v.w;
            }
            float c = 0.f;
#pragma unroll
            for (int i = 0; i < C; ++i) { c += gv[i]; gv[i] = c; }
#pragma unroll
            for (int i4 = 0; i4 < C / 4; ++i4)
                reinterpret_cast<float4*>(cum_s)[i4] = make_float4(gv[4 * i4], gv[4 * i4 + 1], gv[4 * i4 + 2], gv[4 * i4 + 3]);
        }
        __syncthreads();
        {
            const float cumC = cum_s[C - 1];
            if (ln < 8) {
                const int r = warp * 8 + ln;
                const float qi = my_qinv;
                const float e = expf(cum_s[r]);
                ecum_s[r] = e;
                qn_s[r] = __fmul_rn(qi, q_scale);
                qsc_s[r] = __fmul_rn(__fmul_rn(qi, q_scale), e);
                kout_s[r] = __fmul_rn(kinv_s[r], expf(cumC - cum_s[r]));
            }
        }
        __syncthreads();

        // ---- beta v into the right-hand-side tile ------------------------------------------------------
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int i = tid + 256 * u, r = i >> 4, cc = i & 15;
            float vf[8];
            unpack8f(vraw[u], vf);
            const float b = beta_s[r];
            float4* xv = reinterpret_cast<float4*>(V_s + r * V_LD + cc * 8);
            xv[0] = make_float4(vf[0] * b, vf[1] * b, vf[2] * b, vf[3] * b);
            xv[1] = make_float4(vf[4] * b, vf[5] * b, vf[6] * b, vf[7] * b);
        }

        // ---- G = K K^T (warps 0-3) and P = Q K^T (warps 4-7), rows 16 (warp & 3).., columns <= row -
        {
            const int mt = warp < 4 ? warp : 7 - warp, m0 = 16 * mt;    // work grows with mt: a scheduler's two warps get mt and 3 - mt
            const bool is_p = warp >= 4;
            const uint32_t a_base = smem_u32(is_p ? Q_s : K_s) + (uint32_t)((m0 + (ln & 15)) * KQ_LD + (ln >> 4) * 8) * 2u;
            const uint32_t b_base = smem_u32(K_s) + (uint32_t)(((ln & 7) + (ln >> 4) * 8) * KQ_LD + ((ln >> 3) & 1) * 8) * 2u;
            float acc[4][2][4];
#pragma unroll
            for (int np = 0; np < 4; ++np)
#pragma unroll
                for (int e = 0; e < 4; ++e) { acc[np][0][e] = 0.f; acc[np][1][e] = 0.f; }
#pragma unroll
            for (int ks = 0; ks < 8; ++ks) {
                uint32_t a[4];
                ldsm4(a, a_base + ks * 32);
#pragma unroll
                for (int np = 0; np < 4; ++np) {
                    if (np <= mt) {
                        uint32_t b[4];
                        ldsm4(b, b_base + (uint32_t)(np * 16 * KQ_LD) * 2u + ks * 32);
                        mma_bf16_16816(acc[np][0], a, b[0], b[1]);
                        mma_bf16_16816(acc[np][1], a, b[2], b[3]);
                    }
                }
            }
            float* dst = is_p ? Int_s : Tri_s;
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                const int i = m0 + g + 8 * half;
                const float ci = cum_s[i];
                const float gi = __fmul_rn(beta_s[i], kinv_s[i]);
#pragma unroll
                for (int np = 0; np < 4; ++np) {
                    if (np <= mt) {
#pragma unroll
                        for (int n2 = 0; n2 < 2; ++n2) {
                            float out2[2];
#pragma unroll
                            for (int e = 0; e < 2; ++e) {
                                const int j = 16 * np + 8 * n2 + 2 * t + e;
                                const float a = acc[np][n2][2 * half + e];
                                float v = 0.f;
                                if (j <= i) {
                                    const float dec = expf(ci - cum_s[j]);
                                    const float kj = kinv_s[j];
                                    if (is_p) v = a * kj * dec;              // times the q row scale below
                                    else if (j < i) v = a * gi * kj * dec;
                                }
                                out2[e] = v;
                            }
                            *reinterpret_cast<float2*>(dst + i * T_LD + 16 * np + 8 * n2 + 2 * t) = make_float2(out2[0], out2[1]);
                        }
                    }
                }
            }
        }
        asm volatile("cp.async.wait_all;\n" ::: "memory");          // this thread's part of the state has landed
        __syncthreads();

        // ---- the four 16 x 16 diagonal blocks of I + L, inverted by forward substitution ----------------
        if (tid < 64) {
            const int b16 = (tid >> 4) * 16, c = tid & 15;            // thread = column c of block b16 / 16
            float x[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) x[i] = 0.f;                  // a group of four may reach past row i: times zero
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                float a0 = (i == c) ? 1.f : 0.f, a1 = 0.f;
#pragma unroll
                for (int j4 = 0; j4 < 4; ++j4) {                      // entries at and right of the diagonal are zero
                    if (4 * j4 >= i) break;
                    const float4 tr = *reinterpret_cast<const float4*>(Tri_s + (b16 + i) * T_LD + b16 + 4 * j4);
                    a0 -= tr.x * x[4 * j4];
                    a1 -= tr.y * x[4 * j4 + 1];
                    a0 -= tr.z * x[4 * j4 + 2];
                    a1 -= tr.w * x[4 * j4 + 3];
                }
                x[i] = a0 + a1;
            }
#pragma unroll
            for (int i = 0; i < 16; ++i) Tinv_s[(b16 + i) * T_LD + b16 + c] = x[i];
        }

        // ---- q~ S and k~ S in one pass over the state (q~, k~: the raw bf16 rows; warp = 16 rows x 64 columns);
        // then the right-hand side  beta v - (beta e^cum / |k|) (k~ S).  With T = inv(I + L) this gives
        // v_new = T (beta v) - T (beta e^cum k_hat) S  without ever forming  T (beta e^cum k_hat) ------------
        const int mt = warp < 4 ? warp : 7 - warp, m0 = 16 * mt, nb = (warp >> 2) * 64;
        float acc[8][4];                                              // q~ S: kept until the output stage
        {
            float acck[8][4];
#pragma unroll
            for (int nt = 0; nt < 8; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) { acc[nt][e] = 0.f; acck[nt][e] = 0.f; }
            const uint16_t* Qr = Q_s + (m0 + g) * KQ_LD + t;
            const uint16_t* Kr = K_s + (m0 + g) * KQ_LD + t;
            const float* Br = S_s + t * S_LD + nb + g;
#pragma unroll 2
            for (int ks = 0; ks < 16; ++ks) {
                const int k0 = 8 * ks;
                uint32_t aq[4], ak[4];
                aq[0] = (uint32_t)Qr[k0] << 16;
                aq[1] = (uint32_t)Qr[8 * KQ_LD + k0] << 16;
                aq[2] = (uint32_t)Qr[k0 + 4] << 16;
                aq[3] = (uint32_t)Qr[8 * KQ_LD + k0 + 4] << 16;
                ak[0] = (uint32_t)Kr[k0] << 16;
                ak[1] = (uint32_t)Kr[8 * KQ_LD + k0] << 16;
                ak[2] = (uint32_t)Kr[k0 + 4] << 16;
                ak[3] = (uint32_t)Kr[8 * KQ_LD + k0 + 4] << 16;
                mma_row_pair<8>(acc, acck, aq, ak, Br + k0 * S_LD, Br + (k0 + 4) * S_LD);
            }
            const int r0 = m0 + g, r1 = r0 + 8;
            const float kb0 = __fmul_rn(__fmul_rn(kinv_s[r0], beta_s[r0]), ecum_s[r0]);
            const float kb1 = __fmul_rn(__fmul_rn(kinv_s[r1], beta_s[r1]), ecum_s[r1]);
#pragma unroll
            for (int nt = 0; nt < 8; ++nt) {
                float2* p0 = reinterpret_cast<float2*>(V_s + r0 * V_LD + nb + 8 * nt + 2 * t);
                float2* p1 = reinterpret_cast<float2*>(V_s + r1 * V_LD + nb + 8 * nt + 2 * t);
                float2 v0 = *p0, v1 = *p1;
                v0.x -= kb0 * acck[nt][0]; v0.y -= kb0 * acck[nt][1];
                v1.x -= kb1 * acck[nt][2]; v1.y -= kb1 * acck[nt][3];
                *p0 = v0; *p1 = v1;
            }
        }
        __syncthreads();

        // ---- v_new = T rhs by block rows: X_b = inv(D_b) (B_b - sum_{c<b} L_bc X_c); a warp owns 16 columns ----
        {
            float* X = V_s + 16 * warp;
            constexpr int ld = V_LD;
#pragma unroll 1
            for (int b = 0; b < 4; ++b) {
                float r[2][4], ra[2][4], rb[2][4];
#pragma unroll
                for (int nt = 0; nt < 2; ++nt) {
                    const float2 v0 = *reinterpret_cast<const float2*>(X + (16 * b + g) * ld + 8 * nt + 2 * t);
                    const float2 v1 = *reinterpret_cast<const float2*>(X + (16 * b + g + 8) * ld + 8 * nt + 2 * t);
                    r[nt][0] = v0.x; r[nt][1] = v0.y; r[nt][2] = v1.x; r[nt][3] = v1.y;
#pragma unroll
                    for (int e = 0; e < 4; ++e) { ra[nt][e] = 0.f; rb[nt][e] = 0.f; }
                }
                const float* Lr = Tri_s + (16 * b + g) * T_LD + t;
#pragma unroll 2
                for (int k0 = 0; k0 < 16 * b; k0 += 8) {              // minus L_bc X_c: the A fragment carries the sign
                    uint32_t ahi[4], alo[4];
                    split_tf32(-Lr[k0], ahi[0], alo[0]);
                    split_tf32(-Lr[8 * T_LD + k0], ahi[1], alo[1]);
                    split_tf32(-Lr[k0 + 4], ahi[2], alo[2]);
                    split_tf32(-Lr[8 * T_LD + k0 + 4], ahi[3], alo[3]);
                    mma_row3<2>(r, ra, rb, ahi, alo, X + (k0 + t) * ld + g, X + (k0 + t + 4) * ld + g);
                }
                __syncwarp();
#pragma unroll
                for (int nt = 0; nt < 2; ++nt) {                      // the residual becomes a B operand: through shared memory
#pragma unroll
                    for (int e = 0; e < 4; ++e) r[nt][e] += ra[nt][e] + rb[nt][e];
                    *reinterpret_cast<float2*>(X + (16 * b + g) * ld + 8 * nt + 2 * t) = make_float2(r[nt][0], r[nt][1]);
                    *reinterpret_cast<float2*>(X + (16 * b + g + 8) * ld + 8 * nt + 2 * t) = make_float2(r[nt][2], r[nt][3]);
#pragma unroll
                    for (int e = 0; e < 4; ++e) { r[nt][e] = 0.f; ra[nt][e] = 0.f; rb[nt][e] = 0.f; }
                }
                __syncwarp();
                const float* Dr = Tinv_s + (16 * b + g) * T_LD + 16 * b + t;
#pragma unroll
                for (int k0 = 0; k0 < 16; k0 += 8) {
                    uint32_t ahi[4], alo[4];
                    split_tf32(Dr[k0], ahi[0], alo[0]);
                    split_tf32(Dr[8 * T_LD + k0], ahi[1], alo[1]);
                    split_tf32(Dr[k0 + 4], ahi[2], alo[2]);
                    split_tf32(Dr[8 * T_LD + k0 + 4], ahi[3], alo[3]);
                    mma_row3<2>(r, ra, rb, ahi, alo, X + (16 * b + k0 + t) * ld + g, X + (16 * b + k0 + t + 4) * ld + g);
                }
                __syncwarp();
#pragma unroll
                for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
                    for (int e = 0; e < 4; ++e) r[nt][e] += ra[nt][e] + rb[nt][e];
                    *reinterpret_cast<float2*>(X + (16 * b + g) * ld + 8 * nt + 2 * t) = make_float2(r[nt][0], r[nt][1]);
                    *reinterpret_cast<float2*>(X + (16 * b + g + 8) * ld + 8 * nt + 2 * t) = make_float2(r[nt][2], r[nt][3]);
                }
                __syncwarp();
            }
        }
        __syncthreads();

        // ---- o = (q row-scaled) S + intra v_new ; gated RMSNorm ; store y -------------------------
        {
            float acc2[8][4];
#pragma unroll
            for (int nt = 0; nt < 8; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) acc2[nt][e] = 0.f;
            // the epilogue's gate and weight values: asked for now, used after the products
            uint32_t zreg[2][8], wreg[8];
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                const int r = m0 + g + 8 * half;
                const uint16_t* zr = pr0 + (size_t)(r < valid ? r : 0) * kGdnProjN + kOffZ + h * 128 + nb + 2 * t;
#pragma unroll
                for (int nt = 0; nt < 8; ++nt) zreg[half][nt] = *reinterpret_cast<const uint32_t*>(zr + 8 * nt);
            }
#pragma unroll
            for (int nt = 0; nt < 8; ++nt) wreg[nt] = *reinterpret_cast<const uint32_t*>(norm_w + nb + 8 * nt + 2 * t);
            // intra rows only reach columns m <= row; rows of this warp end at m0 + 15
            const float* Ir = Int_s + (m0 + g) * T_LD + t;
            const float* Vr = V_s + t * V_LD + nb + g;
#pragma unroll 1
            for (int ks = 0; ks < 2 * mt + 2; ++ks) {
                const int k0 = 8 * ks;
                uint32_t ahi[4], alo[4];
                split_tf32(Ir[k0], ahi[0], alo[0]);
                split_tf32(Ir[8 * T_LD + k0], ahi[1], alo[1]);
                split_tf32(Ir[k0 + 4], ahi[2], alo[2]);
                split_tf32(Ir[8 * T_LD + k0 + 4], ahi[3], alo[3]);
                mma_row<8, false>(acc2, ahi, alo, Vr + k0 * V_LD, Vr + (k0 + 4) * V_LD, 1.f, 1.f);
            }
            // o = e^cum * qinv*scale * (q~ S)  +  qinv*scale * sum_m (q~.k_m kinv_m e^(cum_r-cum_m)) v_new[m]
            const int r0 = m0 + g, r1 = r0 + 8;
            const float qf0 = qsc_s[r0], qn0 = qn_s[r0], qf1 = qsc_s[r1], qn1 = qn_s[r1];
            float ss0 = 0.f, ss1 = 0.f;
#pragma unroll
            for (int nt = 0; nt < 8; ++nt) {
                acc[nt][0] = acc[nt][0] * qf0 + acc2[nt][0] * qn0;
                acc[nt][1] = acc[nt][1] * qf0 + acc2[nt][1] * qn0;
                acc[nt][2] = acc[nt][2] * qf1 + acc2[nt][2] * qn1;
                acc[nt][3] = acc[nt][3] * qf1 + acc2[nt][3] * qn1;
                ss0 += acc[nt][0] * acc[nt][0] + acc[nt][1] * acc[nt][1];
                ss1 += acc[nt][2] * acc[nt][2] + acc[nt][3] * acc[nt][3];
            }
            ss0 += __shfl_xor_sync(0xffffffffu, ss0, 1); ss0 += __shfl_xor_sync(0xffffffffu, ss0, 2);
            ss1 += __shfl_xor_sync(0xffffffffu, ss1, 1); ss1 += __shfl_xor_sync(0xffffffffu, ss1, 2);
            if (t == 0) { red_s[(warp >> 2) * C + r0] = ss0; red_s[(warp >> 2) * C + r1] = ss1; }
            __syncthreads();                  // also: every read of S by this phase is done
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                const int r = half == 0 ? r0 : r1;
                if (r < valid) {
                    const float rinv = rsqrt_acc((red_s[r] + red_s[C + r]) * (1.0f / 128.0f) + kEps);
                    uint16_t* yr = y + ((size_t)lane_id * T + t0 + r) * kValueDim + h * 128 + nb + 2 * t;
#pragma unroll
                    for (int nt = 0; nt < 8; ++nt) {
                        const uint32_t zv = zreg[half][nt], wv = wreg[nt];
                        float n0 = __fmul_rn(acc[nt][2 * half], rinv), n1 = __fmul_rn(acc[nt][2 * half + 1], rinv);
                        n0 = __fmul_rn(lo_bf(wv), n0);
                        n1 = __fmul_rn(hi_bf(wv), n1);
                        const float z0 = lo_bf(zv), z1 = hi_bf(zv);      // SiLU with the fast exp / divide: the bf16 cast hides their 2 ulp
                        *reinterpret_cast<uint32_t*>(yr + 8 * nt) =
                            pack_bf2(__fmul_rn(n0, __fdividef(z0, 1.0f + __expf(-z0))), __fmul_rn(n1, __fdividef(z1, 1.0f + __expf(-z1))));
                    }
                }
            }
        }

        // ---- S = e^cumC S + k_hat^T (e^(cumC - cum) v_new)   (warp: 16 rows of S, all 128 columns) --
        {
            const int d0 = 16 * warp;
            const float cd = expf(cum_s[C - 1]);
            float acc[16][4];
#pragma unroll
            for (int nt = 0; nt < 16; ++nt) {
                const float2 s0 = *reinterpret_cast<const float2*>(S_s + (d0 + g) * S_LD + 8 * nt + 2 * t);
                const float2 s1 = *reinterpret_cast<const float2*>(S_s + (d0 + g + 8) * S_LD + 8 * nt + 2 * t);
                acc[nt][0] = s0.x * cd; acc[nt][1] = s0.y * cd; acc[nt][2] = s1.x * cd; acc[nt][3] = s1.y * cd;
            }
            const uint16_t* Kr = K_s + t * KQ_LD + d0 + g;
            const float* Vr = V_s + t * V_LD + g;
            float (&acc_lo)[8][4] = *reinterpret_cast<float (*)[8][4]>(&acc[0]);
            float (&acc_hi)[8][4] = *reinterpret_cast<float (*)[8][4]>(&acc[8]);
#pragma unroll 2
            for (int ks = 0; ks < 8; ++ks) {
                const int k0 = 8 * ks;
                uint32_t a[4];
                a[0] = (uint32_t)Kr[k0 * KQ_LD] << 16;
                a[1] = (uint32_t)Kr[k0 * KQ_LD + 8] << 16;
                a[2] = (uint32_t)Kr[(k0 + 4) * KQ_LD] << 16;
                a[3] = (uint32_t)Kr[(k0 + 4) * KQ_LD + 8] << 16;
                const float w0 = kout_s[k0 + t], w1 = kout_s[k0 + t + 4];
                mma_row<8, true>(acc_lo, a, a, Vr + k0 * V_LD, Vr + (k0 + 4) * V_LD, w0, w1);
                mma_row<8, true>(acc_hi, a, a, Vr + k0 * V_LD + 64, Vr + (k0 + 4) * V_LD + 64, w0, w1);
            }
#pragma unroll
            for (int nt = 0; nt < 16; ++nt) {
                *reinterpret_cast<float2*>(S_s + (d0 + g) * S_LD + 8 * nt + 2 * t) = make_float2(acc[nt][0], acc[nt][1]);
                *reinterpret_cast<float2*>(S_s + (d0 + g + 8) * S_LD + 8 * nt + 2 * t) = make_float2(acc[nt][2], acc[nt][3]);
            }
        }
        __syncthreads();
    }

    for (int i = tid; i < 128 * 32; i += 256)
        reinterpret_cast<float4*>(S_g)[i] = *reinterpret_cast<const float4*>(S_s + (i >> 5) * S_LD + (i & 31) * 4);
}

// ---- (2'') the chunk scan with its two large products on the 5th-generation tensor cores ------------
// Same algebra and order as gdn_chunk_tc_kernel; what changes is where the two 128-wide products run:
//   (X)  [q~ ; k~] S        128 x 128 x 128   ->  tcgen05.mma, accumulator D_X in tensor memory
//   (Y)  k~^T (kout v_new)  128 x  64 x 128   ->  tcgen05.mma, accumulator D_Y in tensor memory
// Operands are bf16 in shared memory with the 128-byte swizzle.  q~ and k~ ARE bf16 values; an f32 operand
// x (the state, kout v_new) is fed as three bf16 pieces x = p1 + p2 + p3 (p1 = bf16(x), p2 = bf16(x - p1),
// p3 = bf16(x - p1 - p2): 24 significand bits, the remainders are exact in f32), three MMAs per product.
// Layouts: the q / k chunk tile is [128 rows = 64 q tokens | 64 k tokens][128 d_k] as two K-major slabs of
// 64 d_k (16 KiB each); read as A of (X) it is K-major, and its k rows read as A of (Y) (M = d_k, K = token)
// are the same bytes seen MN-major.  The state pieces are [d_k][d_v], MN-major B of (X), two slabs of 64
// d_v; the kout v_new pieces are [token][d_v], MN-major B of (Y).
// The f32 master copy of the state lives in REGISTERS for the whole kernel (thread = one d_k row x 64 d_v
// columns, the layout tcgen05.ld returns D_Y in), so shared memory holds only operands: the pieces of S
// are dead between the end of (X) and the state update, and that space carries q~ S (handed from tensor
// memory to the mma.sync fragment layout of the output stage) and the pieces of kout v_new meanwhile.
// (X) is issued ahead of the diagonal inverses (64 threads' work) and runs beside them; (Y) is issued after the
// solve and runs under the output stage.  The 64 x 64 products
// (G, P, the blocked solve, intra) stay on warp-level mma as in gdn_chunk_tc_kernel.
// Both completion waits are bounded; on expiry the CTA raises the status word, frees its tensor memory and
// leaves without storing the state.
constexpr int U_AT_BYTES = 2 * 128 * 128;                       // q | k chunk tile, two slabs
constexpr int U_SP_BYTES = 3 * 2 * 128 * 128;                   // three pieces of S, two d_v slabs each
constexpr int U_QS_LD = 132;                                    // f32 row stride of q~ S and k~ S (= 4 mod 32: a thread per row stores 16 bytes conflict-free)
constexpr int U_WP_OFF = 36864;                                 // kout v_new pieces inside the S-piece space (behind q~ S; k~ S is dead by then)
constexpr int U_WP_BYTES = 3 * 2 * 64 * 128;
static_assert(C * U_QS_LD * 4 <= U_WP_OFF && U_WP_OFF + U_WP_BYTES <= U_SP_BYTES && 2 * C * U_QS_LD * 4 <= U_SP_BYTES,
              "aliases fit in the S-piece space");
constexpr size_t kChunkUmmaSmem = 1024 + U_AT_BYTES + U_SP_BYTES + (size_t)C * V_LD * 4 + 3 * (size_t)C * T_LD * 4 +
                                  8 * C * 4 + 2 * C * 4;
static_assert((size_t)128 * U_QS_LD * 4 <= (size_t)C * V_LD * 4 + 3 * (size_t)C * T_LD * 4, "the state's staging copy fits over V / Tri / Int / Tinv");

// byte offset of the 16-byte chunk `ch` (8 d_k values, ch = 0..15) of row `row` in the q | k tile
__device__ __forceinline__ uint32_t at_off(int row, int ch) {
    return (uint32_t)((ch >> 3) * 16384 + row * 128 + (((ch & 7) ^ (row & 7)) << 4));
}
// x = p1 + p2 + p3 in bf16 pieces
__device__ __forceinline__ void split3(float x, float& r1, float& r2, uint16_t& p1, uint16_t& p2, uint16_t& p3) {
    p1 = f2bf(x);
    r1 = __fsub_rn(x, bf2f(p1));
    p2 = f2bf(r1);
    r2 = __fsub_rn(r1, bf2f(p2));
    p3 = f2bf(r2);
}
// eight consecutive f32 values -> one 16-byte chunk of each of the three piece tiles
__device__ __forceinline__ void split3_store8(const float (&v)[8], uint8_t* p1, uint8_t* p2, uint8_t* p3) {
    uint32_t w1[4], w2[4], w3[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        float ra, rb;
        uint16_t a1, a2, a3, b1, b2, b3;
        split3(v[2 * j], ra, rb, a1, a2, a3);
        split3(v[2 * j + 1], ra, rb, b1, b2, b3);
        w1[j] = (uint32_t)a1 | ((uint32_t)b1 << 16);
        w2[j] = (uint32_t)a2 | ((uint32_t)b2 << 16);
        w3[j] = (uint32_t)a3 | ((uint32_t)b3 << 16);
    }
    *reinterpret_cast<uint4*>(p1) = make_uint4(w1[0], w1[1], w1[2], w1[3]);
    *reinterpret_cast<uint4*>(p2) = make_uint4(w2[0], w2[1], w2[2], w2[3]);
    *reinterpret_cast<uint4*>(p3) = make_uint4(w3[0], w3[1], w3[2], w3[3]);
}

__global__ void __launch_bounds__(256, 1)
gdn_chunk_umma_kernel(const uint16_t* __restrict__ proj, const uint16_t* __restrict__ A_log,
                      const uint16_t* __restrict__ dt_bias, const uint16_t* __restrict__ norm_w,
                      float* __restrict__ S0, float* __restrict__ S1, float* __restrict__ S2,
                      const int* __restrict__ sel, uint16_t* __restrict__ y, int T, int* __restrict__ status) {
    extern __shared__ __align__(16) unsigned char smem_chunk[];
    __shared__ __align__(8) unsigned long long bars[2];
    __shared__ uint32_t tmem_base_s;
    const uint32_t base_u = (smem_u32(smem_chunk) + 1023u) & ~1023u;         // the swizzled tiles want 1024-byte alignment
    uint8_t* base_p = smem_chunk + (base_u - smem_u32(smem_chunk));
    uint8_t* AT = base_p;                                                    // q | k tile
    uint8_t* SP = AT + U_AT_BYTES;                                           // S pieces; later q~ S and the kout v_new pieces
    float* QS_s = reinterpret_cast<float*>(SP);                              // [64][132] f32 q~ S, alias
    float* KS_s = QS_s + C * U_QS_LD;                                        // [64][132] f32 k~ S, alias (dead before the pieces below are written)
    uint8_t* WP = SP + U_WP_OFF;                                             // [3][2][64][128 B], alias
    float* V_s = reinterpret_cast<float*>(SP + U_SP_BYTES);                  // [64][136]   beta v, right-hand side, v_new
    float* St_s = V_s;                                                       // [128][132] f32: the state on its way between global memory
                                                                             // (coalesced 16-byte pieces) and the thread-per-row registers;
                                                                             // alias of V_s .. Tinv_s, free at both ends of the kernel
    float* Tri_s = V_s + C * V_LD;                                           // [64][68]
    float* Int_s = Tri_s + C * T_LD;                                         // [64][68]
    float* Tinv_s = Int_s + C * T_LD;                                        // [64][68]   inverses of the diagonal blocks
    float* sc = Tinv_s + C * T_LD;                                           // 8 x [64] row scalars
    float* red_s = sc + 8 * C;                                               // [2][64] sum of squares per column half
    float* cum_s = sc;
    float* beta_s = sc + 64;
    float* kinv_s = sc + 128;
    float* qsc_s = sc + 192;
    float* ecum_s = sc + 256;
    float* kout_s = sc + 320;
    float* g_s = sc + 384;
    float* qn_s = sc + 448;
    const uint32_t at_u = base_u, sp_u = base_u + U_AT_BYTES, wp_u = sp_u + U_WP_OFF;
    const uint32_t bar_x = smem_u32(&bars[0]), bar_y = smem_u32(&bars[1]);

    const int h = blockIdx.x, lane_id = blockIdx.y;
    const int tid = threadIdx.x, warp = tid >> 5, ln = tid & 31;
    const int g = ln >> 2, t = ln & 3;                 // fragment coordinates of this lane
    const int live = sel != nullptr ? sel[lane_id] : 0;
    float* S_g = (live == 0 ? S0 : (live == 1 ? S1 : S2)) + ((size_t)lane_id * kGdnHeads + h) * (kDk * kDv);
    const float negA = -expf(bf2f(A_log[h]));
    const float dtb = bf2f(dt_bias[h]);
    const float q_scale = 0.08838834764831845f;
    // this thread's part of the state and of every tensor-memory accumulator: row (= lane of tensor memory) srow,
    // columns [scol, scol + 64)
    const int srow = 32 * (warp & 3) + ln, scol = 64 * (warp >> 2);
    if (tid == 0) {
        mbar_init(bar_x, 1);
        mbar_init(bar_y, 1);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n"
                     ::"r"(smem_u32(&tmem_base_s)), "r"(256u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    // the state: global -> registers (kept for the whole kernel) -> its three bf16 pieces in shared memory;
    // requested behind the first chunk's q / k rows (below), like every other load of the chunk
    float S[64];
    auto store_state_pieces = [&]() {
        uint8_t* rowp = SP + (warp >> 2) * 16384 + srow * 128;               // slab of this thread's d_v half, row d_k = srow
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            float v[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) v[e] = S[8 * j + e];
            uint8_t* q = rowp + ((j ^ (srow & 7)) << 4);
            split3_store8(v, q, q + 32768, q + 65536);
        }
    };
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_base_s;
    const uint32_t dX = tmem, dY = tmem + 128;
    const uint32_t lane_sel = (uint32_t)(32 * (warp & 3)) << 16;
    constexpr uint32_t IDESC_X = instr_desc(128, 128, 0, 1);                 // A K-major, B MN-major
    constexpr uint32_t IDESC_Y = instr_desc(128, 128, 1, 1);                 // both MN-major
    bool failed = false;

    const int n_chunks = (T + C - 1) / C;
    for (int ck = 0; ck < n_chunks && !failed; ++ck) {
        const int t0 = ck * C;
        const int valid = (T - t0) < C ? (T - t0) : C;
        const uint32_t par = (uint32_t)(ck & 1);
        const uint16_t* pr0 = proj + ((size_t)lane_id * T + t0) * kGdnProjN;

        // ---- q, k rows into the swizzled tile (zero rows past T), v pieces and gate inputs to registers --------
        for (int i = tid; i < C * 16; i += 256) {
            const int r = i >> 4, cc = i & 15;
            const uint16_t* pr = pr0 + (size_t)(r < valid ? r : 0) * kGdnProjN + h * 128 + cc * 8;
            const uint32_t n = r < valid ? 16u : 0u;                // 0 bytes read = 16 bytes of zeros written
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n"
                         ::"r"(at_u + at_off(r, cc)), "l"(pr), "r"(n) : "memory");
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n"
                         ::"r"(at_u + at_off(64 + r, cc)), "l"(pr + 2048), "r"(n) : "memory");
        }
        asm volatile("cp.async.commit_group;\n" ::: "memory");
        uint4 vraw[4];                               // this thread's v pieces, used by the right-hand sides
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int i = tid + 256 * u, r = i >> 4, cc = i & 15;
            vraw[u] = make_uint4(0, 0, 0, 0);
            if (r < valid) vraw[u] = *reinterpret_cast<const uint4*>(pr0 + (size_t)r * kGdnProjN + 4096 + h * 128 + cc * 8);
        }
        float b_in = 0.f, a_in = 0.f;
        if (tid < valid) {
            const uint16_t* pr = pr0 + (size_t)tid * kGdnProjN;
            b_in = bf2f(pr[kOffB + h]);
            a_in = bf2f(pr[kOffA + h]);
        }
        if (ck == 0) {                  // the 64 KiB state, 16-byte pieces in global order, into the padded staging rows
            for (int i = tid; i < 128 * 32; i += 256)
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n"
                             ::"r"(smem_u32(St_s + (i >> 5) * U_QS_LD + (i & 31) * 4)), "l"(S_g + 4 * i) : "memory");
            asm volatile("cp.async.commit_group;\n" ::: "memory");
        }
        if (tid < C) {
            float beta = 0.f, gg = 0.f;
            if (tid < valid) {
                beta = sigmoid_acc(b_in);
                const float sp_in = a_in + dtb;
                const float sp = sp_in > 20.0f ? sp_in : log1pf(expf(sp_in));
                gg = __fmul_rn(negA, sp);
            }
            beta_s[tid] = beta;
            g_s[tid] = gg;
        }
        asm volatile("cp.async.wait_group 0;\n" ::: "memory");
        if (ck == 0) {
            __syncthreads();                                  // every thread's pieces of the staged state have landed
            const float4* sp4 = reinterpret_cast<const float4*>(St_s + srow * U_QS_LD + scol);
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                const float4 v = sp4[i];
                S[4 * i] = v.x; S[4 * i + 1] = v.y; S[4 * i + 2] = v.z; S[4 * i + 3] = v.w;
            }
            store_state_pieces();
        }
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");     // the tile and the S pieces: generic writes -> the MMA's reads
        tc_fence_before();
        __syncthreads();
        // ---- row scalars: L2 norms (warp w takes rows 8w..8w+7), prefix sum of g -----------------
        float my_qs = 0.f, my_ks = 0.f;              // lane rr keeps the sums of row 8 warp + rr
#pragma unroll
        for (int rr = 0; rr < 8; ++rr) {
            const int r = warp * 8 + rr;
            const uint2 kv = *reinterpret_cast<const uint2*>(AT + at_off(64 + r, ln >> 1) + (ln & 1) * 8);
            const uint2 qv = *reinterpret_cast<const uint2*>(AT + at_off(r, ln >> 1) + (ln & 1) * 8);
            float ks = lo_bf(kv.x) * lo_bf(kv.x) + hi_bf(kv.x) * hi_bf(kv.x) + lo_bf(kv.y) * lo_bf(kv.y) + hi_bf(kv.y) * hi_bf(kv.y);
            float qs = lo_bf(qv.x) * lo_bf(qv.x) + hi_bf(qv.x) * hi_bf(qv.x) + lo_bf(qv.y) * lo_bf(qv.y) + hi_bf(qv.y) * hi_bf(qv.y);
            ks = warp_sum(ks);
            qs = warp_sum(qs);
            if (ln == rr) { my_ks = ks; my_qs = qs; }
        }
        float my_qinv = 0.f;
        if (ln < 8) {
            my_qinv = rsqrt_acc(my_qs + 1e-6f);
            kinv_s[warp * 8 + ln] = rsqrt_acc(my_ks + 1e-6f);
        }
        if (tid == 32) {                     // sequential like the reference's cumsum, but from registers (not the MMA-issuing thread)
            float gv[C];
#pragma unroll
            for (int i4 = 0; i4 < C / 4; ++i4) {
                const float4 v = reinterpret_cast<const float4*>(g_s)[i4];
                gv[4 * i4] = v.x; gv[4 * i4 + 1] = v.y; gv[4 * i4 + 2] = v.z; gv[4 * i4 + 3] = v.w;
            }
            float c = 0.f;
#pragma unroll
            for (int i = 0; i < C; ++i) { c += gv[i]; gv[i] = c; }
#pragma unroll
            for (int i4 = 0; i4 < C / 4; ++i4)
                reinterpret_cast<float4*>(cum_s)[i4] = make_float4(gv[4 * i4], gv[4 * i4 + 1], gv[4 * i4 + 2], gv[4 * i4 + 3]);
        }
        __syncthreads();
        {
            const float cumC = cum_s[C - 1];
            if (ln < 8) {
                const int r = warp * 8 + ln;
                const float qi = my_qinv;
                const float e = expf(cum_s[r]);
                ecum_s[r] = e;
                qn_s[r] = __fmul_rn(qi, q_scale);
                qsc_s[r] = __fmul_rn(__fmul_rn(qi, q_scale), e);
                kout_s[r] = __fmul_rn(kinv_s[r], expf(cumC - cum_s[r]));
            }
        }
        __syncthreads();
        // ---- beta v into the right-hand-side tile ------------------------------------------------------
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int i = tid + 256 * u, r = i >> 4, cc = i & 15;
            float vf[8];
            unpack8f(vraw[u], vf);
            const float b = beta_s[r];
            float4* xv = reinterpret_cast<float4*>(V_s + r * V_LD + cc * 8);
            xv[0] = make_float4(vf[0] * b, vf[1] * b, vf[2] * b, vf[3] * b);
            xv[1] = make_float4(vf[4] * b, vf[5] * b, vf[6] * b, vf[7] * b);
        }

        // ---- G = K K^T (warps 0-3) and P = Q K^T (warps 4-7), rows 16 (warp & 3).., columns <= row -
        {
            const int mt = warp < 4 ? warp : 7 - warp, m0 = 16 * mt;    // work grows with mt: a scheduler's two warps get mt and 3 - mt
            const bool is_p = warp >= 4;
            const int arow = (is_p ? 0 : 64) + m0 + (ln & 15);
            const int brow0 = 64 + (ln & 7) + (ln >> 4) * 8;
            float acc[4][2][4];
#pragma unroll
            for (int np = 0; np < 4; ++np)
#pragma unroll
                for (int e = 0; e < 4; ++e) { acc[np][0][e] = 0.f; acc[np][1][e] = 0.f; }
#pragma unroll
            for (int ks = 0; ks < 8; ++ks) {
                uint32_t a[4];
                ldsm4(a, at_u + at_off(arow, 2 * ks + (ln >> 4)));
#pragma unroll
                for (int np = 0; np < 4; ++np) {
                    if (np <= mt) {
                        uint32_t b[4];
                        ldsm4(b, at_u + at_off(brow0 + 16 * np, 2 * ks + ((ln >> 3) & 1)));
                        mma_bf16_16816(acc[np][0], a, b[0], b[1]);
                        mma_bf16_16816(acc[np][1], a, b[2], b[3]);
                    }
                }
            }
            float* dst = is_p ? Int_s : Tri_s;
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                const int i = m0 + g + 8 * half;
                const float ci = cum_s[i];
                const float gi = __fmul_rn(beta_s[i], kinv_s[i]);
#pragma unroll
                for (int np = 0; np < 4; ++np) {
                    if (np <= mt) {
#pragma unroll
                        for (int n2 = 0; n2 < 2; ++n2) {
                            float out2[2];
#pragma unroll
                            for (int e = 0; e < 2; ++e) {
                                const int j = 16 * np + 8 * n2 + 2 * t + e;
                                const float a = acc[np][n2][2 * half + e];
                                float v = 0.f;
                                if (j <= i) {
                                    const float dec = expf(ci - cum_s[j]);
                                    const float kj = kinv_s[j];
                                    if (is_p) v = a * kj * dec;              // times the q row scale below
                                    else if (j < i) v = a * gi * kj * dec;
                                }
                                out2[e] = v;
                            }
                            *reinterpret_cast<float2*>(dst + i * T_LD + 16 * np + 8 * n2 + 2 * t) = make_float2(out2[0], out2[1]);
                        }
                    }
                }
            }
        }
        __syncthreads();
        // ---- (X) [q~ ; k~] S: issued here, by a thread of a warp that has no part in the diagonal inverses below,
        // so that the product (about 1,600 cycles of tensor time, during which its issuing thread is held) runs
        // beside them instead of holding one warp back in a phase every warp works in ------------------------------
        if (tid == 0) {
            tc_fence_after();
#pragma unroll
            for (int pc = 0; pc < 3; ++pc)
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const uint64_t da = smem_desc_sw128(at_u + (j >> 2) * 16384 + (j & 3) * 32);
                    const uint64_t db = smem_desc_sw128_ex(sp_u + pc * 32768 + j * 2048, 16384, 1024);
                    tc_mma(dX, da, db, IDESC_X, (pc | j) != 0 ? 1u : 0u);
                }
            tc_commit(bar_x);
        }

        // ---- the four 16 x 16 diagonal blocks of I + L, inverted by forward substitution ----------------
        if (tid >= 64 && tid < 128) {
            const int u = tid - 64;
            const int b16 = (u >> 4) * 16, c = u & 15;                // thread = column c of block b16 / 16
            float x[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) x[i] = 0.f;                  // a group of four may reach past row i: times zero
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                float a0 = (i == c) ? 1.f : 0.f, a1 = 0.f;
#pragma unroll
                for (int j4 = 0; j4 < 4; ++j4) {                      // entries at and right of the diagonal are zero
                    if (4 * j4 >= i) break;
                    const float4 tr = *reinterpret_cast<const float4*>(Tri_s + (b16 + i) * T_LD + b16 + 4 * j4);
                    a0 -= tr.x * x[4 * j4];
                    a1 -= tr.y * x[4 * j4 + 1];
                    a0 -= tr.z * x[4 * j4 + 2];
                    a1 -= tr.w * x[4 * j4 + 3];
                }
                x[i] = a0 + a1;
            }
#pragma unroll
            for (int i = 0; i < 16; ++i) Tinv_s[(b16 + i) * T_LD + b16 + c] = x[i];
        }
        // ---- (X) done: k~ S rows fold into the right-hand side, q~ S rows go to shared memory for the output stage.
        // With T = inv(I + L):  v_new = T (beta v) - T (beta e^cum k_hat) S  without ever forming T (beta e^cum k_hat)
        if (!__syncthreads_and(mbar_wait_bounded(bar_x, par))) { failed = true; break; }
        tc_fence_after();
        {
            // tensor memory -> shared memory, thread = row: q~ S (tokens 0..63) and k~ S behind it (one buffer of 128 rows)
            float4* dp = reinterpret_cast<float4*>(QS_s + srow * U_QS_LD + scol);
            uint32_t rv[32];
            tmem_ld32(dX + lane_sel + scol, rv);
#pragma unroll
            for (int i = 0; i < 8; ++i) dp[i] = make_float4(__uint_as_float(rv[4 * i]), __uint_as_float(rv[4 * i + 1]),
                                                           __uint_as_float(rv[4 * i + 2]), __uint_as_float(rv[4 * i + 3]));
            tmem_ld32(dX + lane_sel + scol + 32, rv);
#pragma unroll
            for (int i = 0; i < 8; ++i) dp[8 + i] = make_float4(__uint_as_float(rv[4 * i]), __uint_as_float(rv[4 * i + 1]),
                                                               __uint_as_float(rv[4 * i + 2]), __uint_as_float(rv[4 * i + 3]));
        }
        tc_fence_before();
        __syncthreads();
        // right-hand side  beta v - (beta e^cum / |k|) (k~ S), row-major over the tile (conflict-free, coalesced)
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const int i = tid + 256 * u, r = i >> 5, c4 = (i & 31) * 4;
            const float kb = __fmul_rn(__fmul_rn(kinv_s[r], beta_s[r]), ecum_s[r]);
            const float4 ks4 = *reinterpret_cast<const float4*>(KS_s + r * U_QS_LD + c4);
            float4* vp = reinterpret_cast<float4*>(V_s + r * V_LD + c4);
            float4 v = *vp;
            v.x -= kb * ks4.x; v.y -= kb * ks4.y; v.z -= kb * ks4.z; v.w -= kb * ks4.w;
            *vp = v;
        }
        __syncthreads();
        // ---- v_new = T rhs by block rows: X_b = inv(D_b) (B_b - sum_{c<b} L_bc X_c); a warp owns 16 columns ----
        {
            float* X = V_s + 16 * warp;
            constexpr int ld = V_LD;
#pragma unroll 1
            for (int b = 0; b < 4; ++b) {
                float r[2][4], ra[2][4], rb[2][4];
#pragma unroll
                for (int nt = 0; nt < 2; ++nt) {
                    const float2 v0 = *reinterpret_cast<const float2*>(X + (16 * b + g) * ld + 8 * nt + 2 * t);
                    const float2 v1 = *reinterpret_cast<const float2*>(X + (16 * b + g + 8) * ld + 8 * nt + 2 * t);
                    r[nt][0] = v0.x; r[nt][1] = v0.y; r[nt][2] = v1.x; r[nt][3] = v1.y;
#pragma unroll
                    for (int e = 0; e < 4; ++e) { ra[nt][e] = 0.f; rb[nt][e] = 0.f; }
                }
                const float* Lr = Tri_s + (16 * b + g) * T_LD + t;
#pragma unroll 2
                for (int k0 = 0; k0 < 16 * b; k0 += 8) {              // minus L_bc X_c: the A fragment carries the sign
                    uint32_t ahi[4], alo[4];
                    split_tf32(-Lr[k0], ahi[0], alo[0]);
                    split_tf32(-Lr[8 * T_LD + k0], ahi[1], alo[1]);
                    split_tf32(-Lr[k0 + 4], ahi[2], alo[2]);
                    split_tf32(-Lr[8 * T_LD + k0 + 4], ahi[3], alo[3]);
                    mma_row3<2>(r, ra, rb, ahi, alo, X + (k0 + t) * ld + g, X + (k0 + t + 4) * ld + g);
                }
                __syncwarp();
#pragma unroll
                for (int nt = 0; nt < 2; ++nt) {                      // the residual becomes a B operand: through shared memory
#pragma unroll
                    for (int e = 0; e < 4; ++e) r[nt][e] += ra[nt][e] + rb[nt][e];
                    *reinterpret_cast<float2*>(X + (16 * b + g) * ld + 8 * nt + 2 * t) = make_float2(r[nt][0], r[nt][1]);
                    *reinterpret_cast<float2*>(X + (16 * b + g + 8) * ld + 8 * nt + 2 * t) = make_float2(r[nt][2], r[nt][3]);
#pragma unroll
                    for (int e = 0; e < 4; ++e) { r[nt][e] = 0.f; ra[nt][e] = 0.f; rb[nt][e] = 0.f; }
                }
                __syncwarp();
                const float* Dr = Tinv_s + (16 * b + g) * T_LD + 16 * b + t;
#pragma unroll
                for (int k0 = 0; k0 < 16; k0 += 8) {
                    uint32_t ahi[4], alo[4];
                    split_tf32(Dr[k0], ahi[0], alo[0]);
                    split_tf32(Dr[8 * T_LD + k0], ahi[1], alo[1]);
                    split_tf32(Dr[k0 + 4], ahi[2], alo[2]);
                    split_tf32(Dr[8 * T_LD + k0 + 4], ahi[3], alo[3]);
                    mma_row3<2>(r, ra, rb, ahi, alo, X + (16 * b + k0 + t) * ld + g, X + (16 * b + k0 + t + 4) * ld + g);
                }
                __syncwarp();
#pragma unroll
                for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
                    for (int e = 0; e < 4; ++e) r[nt][e] += ra[nt][e] + rb[nt][e];
                    *reinterpret_cast<float2*>(X + (16 * b + g) * ld + 8 * nt + 2 * t) = make_float2(r[nt][0], r[nt][1]);
                    *reinterpret_cast<float2*>(X + (16 * b + g + 8) * ld + 8 * nt + 2 * t) = make_float2(r[nt][2], r[nt][3]);
                }
                __syncwarp();
            }
        }
        __syncthreads();
        // ---- the three bf16 pieces of kout v_new [token][d_v] (thread = 8 tokens' worth of one 32-value strip) ----
        {
            // 64 tokens x 16 chunks of 8 d_v = 1024 chunks, four per thread
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int i = tid + 256 * u, r = i >> 4, cc = i & 15;
                const float w = kout_s[r];
                const float4 a = *reinterpret_cast<const float4*>(V_s + r * V_LD + cc * 8);
                const float4 b = *reinterpret_cast<const float4*>(V_s + r * V_LD + cc * 8 + 4);
                const float v[8] = {a.x * w, a.y * w, a.z * w, a.w * w, b.x * w, b.y * w, b.z * w, b.w * w};
                uint8_t* q = WP + (cc >> 3) * 8192 + r * 128 + (((cc & 7) ^ (r & 7)) << 4);
                split3_store8(v, q, q + 16384, q + 32768);
            }
        }
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
        tc_fence_before();
        __syncthreads();
        // ---- (Y) k~^T (kout v_new), issued now, waited for after the output stage ------------------------------
        if (tid == 0) {
            tc_fence_after();
#pragma unroll
            for (int pc = 0; pc < 3; ++pc)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const uint64_t da = smem_desc_sw128_ex(at_u + 64 * 128 + j * 2048, 16384, 1024);     // the k rows, seen [token][d_k]
                    const uint64_t db = smem_desc_sw128_ex(wp_u + pc * 16384 + j * 2048, 8192, 1024);
                    tc_mma(dY, da, db, IDESC_Y, (pc | j) != 0 ? 1u : 0u);
                }
            tc_commit(bar_y);
        }
        // ---- o = (q row-scaled) S + intra v_new ; gated RMSNorm ; store y -------------------------
        const int mt = warp < 4 ? warp : 7 - warp, m0 = 16 * mt, nb = (warp >> 2) * 64;
        {
            float acc[8][4], acc2[8][4];
#pragma unroll
            for (int nt = 0; nt < 8; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) acc2[nt][e] = 0.f;
            // the epilogue's gate and weight values: asked for now, used after the products
            uint32_t zreg[2][8], wreg[8];
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                const int r = m0 + g + 8 * half;
                const uint16_t* zr = pr0 + (size_t)(r < valid ? r : 0) * kGdnProjN + kOffZ + h * 128 + nb + 2 * t;
#pragma unroll
                for (int nt = 0; nt < 8; ++nt) zreg[half][nt] = *reinterpret_cast<const uint32_t*>(zr + 8 * nt);
            }
#pragma unroll
            for (int nt = 0; nt < 8; ++nt) wreg[nt] = *reinterpret_cast<const uint32_t*>(norm_w + nb + 8 * nt + 2 * t);
            // intra rows only reach columns m <= row; rows of this warp end at m0 + 15
            const float* Ir = Int_s + (m0 + g) * T_LD + t;
            const float* Vr = V_s + t * V_LD + nb + g;
#pragma unroll 1
            for (int ks = 0; ks < 2 * mt + 2; ++ks) {
                const int k0 = 8 * ks;
                uint32_t ahi[4], alo[4];
                split_tf32(Ir[k0], ahi[0], alo[0]);
                split_tf32(Ir[8 * T_LD + k0], ahi[1], alo[1]);
                split_tf32(Ir[k0 + 4], ahi[2], alo[2]);
                split_tf32(Ir[8 * T_LD + k0 + 4], ahi[3], alo[3]);
                mma_row<8, false>(acc2, ahi, alo, Vr + k0 * V_LD, Vr + (k0 + 4) * V_LD, 1.f, 1.f);
            }
            // o = e^cum * qinv*scale * (q~ S)  +  qinv*scale * sum_m (q~.k_m kinv_m e^(cum_r-cum_m)) v_new[m]
            const int r0 = m0 + g, r1 = r0 + 8;
#pragma unroll
            for (int nt = 0; nt < 8; ++nt) {
                const float2 a0 = *reinterpret_cast<const float2*>(QS_s + r0 * U_QS_LD + nb + 8 * nt + 2 * t);
                const float2 a1 = *reinterpret_cast<const float2*>(QS_s + r1 * U_QS_LD + nb + 8 * nt + 2 * t);
                acc[nt][0] = a0.x; acc[nt][1] = a0.y; acc[nt][2] = a1.x; acc[nt][3] = a1.y;
            }
            const float qf0 = qsc_s[r0], qn0 = qn_s[r0], qf1 = qsc_s[r1], qn1 = qn_s[r1];
            float ss0 = 0.f, ss1 = 0.f;
#pragma unroll
            for (int nt = 0; nt < 8; ++nt) {
                acc[nt][0] = acc[nt][0] * qf0 + acc2[nt][0] * qn0;
                acc[nt][1] = acc[nt][1] * qf0 + acc2[nt][1] * qn0;
                acc[nt][2] = acc[nt][2] * qf1 + acc2[nt][2] * qn1;
                acc[nt][3] = acc[nt][3] * qf1 + acc2[nt][3] * qn1;
                ss0 += acc[nt][0] * acc[nt][0] + acc[nt][1] * acc[nt][1];
                ss1 += acc[nt][2] * acc[nt][2] + acc[nt][3] * acc[nt][3];
            }
            ss0 += __shfl_xor_sync(0xffffffffu, ss0, 1); ss0 += __shfl_xor_sync(0xffffffffu, ss0, 2);
            ss1 += __shfl_xor_sync(0xffffffffu, ss1, 1); ss1 += __shfl_xor_sync(0xffffffffu, ss1, 2);
            if (t == 0) { red_s[(warp >> 2) * C + r0] = ss0; red_s[(warp >> 2) * C + r1] = ss1; }
            __syncthreads();
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                const int r = half == 0 ? r0 : r1;
                if (r < valid) {
                    const float rinv = rsqrt_acc((red_s[r] + red_s[C + r]) * (1.0f / 128.0f) + kEps);
                    uint16_t* yr = y + ((size_t)lane_id * T + t0 + r) * kValueDim + h * 128 + nb + 2 * t;
#pragma unroll
                    for (int nt = 0; nt < 8; ++nt) {
                        const uint32_t zv = zreg[half][nt], wv = wreg[nt];
                        float n0 = __fmul_rn(acc[nt][2 * half], rinv), n1 = __fmul_rn(acc[nt][2 * half + 1], rinv);
                        n0 = __fmul_rn(lo_bf(wv), n0);
                        n1 = __fmul_rn(hi_bf(wv), n1);
                        const float z0 = lo_bf(zv), z1 = hi_bf(zv);      // SiLU with the fast exp / divide: the bf16 cast hides their 2 ulp
                        *reinterpret_cast<uint32_t*>(yr + 8 * nt) =
                            pack_bf2(__fmul_rn(n0, __fdividef(z0, 1.0f + __expf(-z0))), __fmul_rn(n1, __fdividef(z1, 1.0f + __expf(-z1))));
                    }
                }
            }
        }
        // ---- (Y) done: S = e^cumC S + D_Y in registers; its pieces for the next chunk ---------------------------
        if (!__syncthreads_and(mbar_wait_bounded(bar_y, par))) { failed = true; break; }
        tc_fence_after();
        {
            const float cd = expf(cum_s[C - 1]);
            uint32_t rv[32];
            tmem_ld32(dY + lane_sel + scol, rv);
#pragma unroll
            for (int i = 0; i < 32; ++i) S[i] = __fmaf_rn(S[i], cd, __uint_as_float(rv[i]));
            tmem_ld32(dY + lane_sel + scol + 32, rv);
#pragma unroll
            for (int i = 0; i < 32; ++i) S[32 + i] = __fmaf_rn(S[32 + i], cd, __uint_as_float(rv[i]));
        }
        if (ck + 1 < n_chunks) store_state_pieces();         // every read of q~ S and of the kout v_new pieces is behind the barrier above
        tc_fence_before();
        __syncthreads();
    }
    if (failed) {
        if (tid == 0 && status != nullptr) atomicExch(status, 8);
    } else {
        float4* sp4 = reinterpret_cast<float4*>(St_s + srow * U_QS_LD + scol);
#pragma unroll
        for (int i = 0; i < 16; ++i) sp4[i] = make_float4(S[4 * i], S[4 * i + 1], S[4 * i + 2], S[4 * i + 3]);
        __syncthreads();
        for (int i = tid; i < 128 * 32; i += 256)
            reinterpret_cast<float4*>(S_g)[i] = *reinterpret_cast<const float4*>(St_s + (i >> 5) * U_QS_LD + (i & 31) * 4);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(256u) : "memory");
    }
}

}  // namespace

// Fills the SiLU table of the current device on `st` (once per device; an engine does it at creation,
// a bare operator call at its first use, ordered ahead of the conv pass on the same stream).
cudaError_t gdn_chunk_init(cudaStream_t st) {
    static bool table_done[64] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
    if (table_done[dev]) return cudaSuccess;
    silu_table_kernel<<<256, 256, 0, st>>>();
    e = cudaGetLastError();
    if (e == cudaSuccess) table_done[dev] = true;
    return e;
}

cudaError_t launch_gdn_chunked(const GdnParams& p, cudaStream_t st) {
    if (p.lanes <= 0 || p.T <= 0 || p.lanes > 65535 || p.checkpoint) return cudaErrorInvalidValue;
    {
        static bool tc_done[kMaxDevices] = {false}, umma_done[kMaxDevices] = {false};     // per device
        cudaError_t e = opt_in_smem(gdn_chunk_tc_kernel, kChunkTcSmem, tc_done);
        if (e == cudaSuccess) e = opt_in_smem(gdn_chunk_umma_kernel, kChunkUmmaSmem, umma_done);
        if (e != cudaSuccess) return e;
    }
    {
        cudaError_t e = gdn_chunk_init(st);         // no-op once this device's table is filled
        if (e != cudaSuccess) return e;
    }
    gdn_conv_prep_kernel<<<dim3(p.lanes, kConvCh / 1024), 128, 0, st>>>(const_cast<uint16_t*>(p.proj), p.conv_w, p.win[0],
                                                                  p.win[1], p.win[2], p.sel, p.T);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    // Q35_GDN_CHUNK=mma: every product on warp-level mma (the cross-check form); default: the two large products on
    // tcgen05 (read per call: a prefill body, not a hot loop)
    const char* env = std::getenv("Q35_GDN_CHUNK");
    if (env != nullptr && env[0] == 'm')
        gdn_chunk_tc_kernel<<<dim3(kGdnHeads, p.lanes), 256, kChunkTcSmem, st>>>(p.proj, p.A_log, p.dt_bias, p.norm_w,
                                                                                p.S[0], p.S[1], p.S[2], p.sel, p.y, p.T);
    else
        gdn_chunk_umma_kernel<<<dim3(kGdnHeads, p.lanes), 256, kChunkUmmaSmem, st>>>(p.proj, p.A_log, p.dt_bias, p.norm_w,
                                                                                    p.S[0], p.S[1], p.S[2], p.sel, p.y, p.T, p.status);
    return cudaGetLastError();
}

}  // namespace q35
