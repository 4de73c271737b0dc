// Batched bf16 projections  out[rows][N] = x[rows][K] . W[N][K]^T  (f32 accumulate, one bf16
// rounding), with the SwiGLU and the lowest-id argmax epilogues fused in.
//
// Two forms:
//   * rows <= 16  : weight-streaming form.  A CTA owns 8*NB weight rows, its 8 warps split K, every
//     thread streams its slice of the weight rows with 16-byte loads issued up front and feeds
//     them to the tensor cores as the B operand of m16n8k16 (x rows are the A operand, so up to
//     16 lanes ride along for free).  Bound by HBM (weights are read exactly once).
//   * rows  > 16  : tiled form.  cp.async multi-stage pipeline into XOR-swizzled shared memory,
//     ldmatrix + m16n8k16, tile BM x BN chosen so that the grid covers the 148 SMs.
// Replaces the reference's proj_group_rows / mlp_gateup / mlp_down / lm_head_gemv_* launchers
// (engine/kernels.h:183-297,363-374,939-945) and its library GEMM route.
#include <cstdlib>

#include "q35_common.cuh"

namespace q35 {

__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                         uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
        "{%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// SwiGLU with the reference's three roundings (speccheck/specimpl.py:400-407):
// g = bf16(dot), u = bf16(dot), act = bf16( bf16(silu(g)) * u ).
__device__ __forceinline__ uint16_t swiglu_bf16(float gate_acc, float up_acc) {
    const float g = bfround(gate_acc);
    const float u = bfround(up_acc);
    const float s = bfround(silu_acc(g));
    return f2bf(s * u);
}

__device__ __forceinline__ uint4 ldg16(const uint16_t* p) {
    return __ldg(reinterpret_cast<const uint4*>(p));
}

// eight residual values -> bf16( (v * inv) * (1 + w) ), the zero-centred RMSNorm's element rule
__device__ __forceinline__ uint32_t norm2(uint32_t v, float inv, uint32_t w) {
    return pack_bf2(__fmul_rn(__fmul_rn(lo_bf(v), inv), 1.0f + lo_bf(w)),
                    __fmul_rn(__fmul_rn(hi_bf(v), inv), 1.0f + hi_bf(w)));
}
__device__ __forceinline__ float sumsq8(const uint4& v) {
    float a = lo_bf(v.x) * lo_bf(v.x);
    a += hi_bf(v.x) * hi_bf(v.x);
    a += lo_bf(v.y) * lo_bf(v.y); a += hi_bf(v.y) * hi_bf(v.y);
    a += lo_bf(v.z) * lo_bf(v.z); a += hi_bf(v.z) * hi_bf(v.z);
    a += lo_bf(v.w) * lo_bf(v.w); a += hi_bf(v.w) * hi_bf(v.w);
    return a;
}
__device__ __forceinline__ uint4 norm8(const uint4& v, float inv, const uint4& w) {
    return make_uint4(norm2(v.x, inv, w.x), norm2(v.y, inv, w.y), norm2(v.z, inv, w.z), norm2(v.w, inv, w.w));
}

// ------------------------------------------------------------------------------------------------
// rows <= 16: weight-streaming form
// ------------------------------------------------------------------------------------------------
// NORM: the x rows are un-normalised residual rows; the kernel applies the zero-centred RMSNorm
// (weights nw) while it stages them.  Every CTA holds all of x, so it takes the rows' sums of squares
// from its own registers (per thread, then across the four lanes that share a row, then across the
// eight warps in warp order: deterministic) - no extra pass over memory.
// EPI_RESID: `out` is the residual stream [M][N], updated in place: resid = bf16(resid + bf16(dot)).
// pf / pf_bytes: weights of a LATER kernel of the body; the CTAs ask the L2 for them (one slice each)
// as soon as their own loads are issued, so that the later kernel streams from L2 while HBM runs ahead
// of the chain of dependent kernels.
struct GemvExtra {
    const uint16_t* nw;        // NORM: norm weights [K]
    const void* pf;            // optional: bytes to pull into L2
    unsigned long long pf_bytes;
    int trigger_early;         // 1: let the successor start right after this kernel's own wait
};

__device__ __forceinline__ void l2_prefetch_slice(const void* base, unsigned long long total, int part, int n_parts) {
    // slice `part` of n_parts, in pieces of at most 32 KiB (sizes multiples of 16 bytes)
    const unsigned long long per = ((total / n_parts) + 15ull) & ~15ull;
    unsigned long long off = per * part;
    if (off >= total) return;
    unsigned long long left = total - off < per ? total - off : per;
    left &= ~15ull;
    const char* p = static_cast<const char*>(base) + off;
    while (left > 0) {
        const unsigned n = left > 32768ull ? 32768u : (unsigned)left;
        asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;\n" ::"l"(p), "r"(n) : "memory");
        p += n;
        left -= n;
    }
}

template <int K, int NB, int EPI, bool NORM>
__global__ void __launch_bounds__(256, 2)
gemv_rows_kernel(const uint16_t* __restrict__ x, const uint16_t* __restrict__ W, void* __restrict__ out,
                 int M, int N, ArgMax* __restrict__ partials, float* __restrict__ logits, int n_parts,
                 GemvExtra ex) {
    constexpr int KW = K / 8;       // k range of one warp
    constexpr int CH = KW / 32;     // 32-wide k chunks per warp
    constexpr int BATCH = (CH <= 8) ? CH : 7;
    static_assert(CH % BATCH == 0, "chunk batching");
    static_assert(!NORM || CH == BATCH, "the normalising form stages all of x in one batch");
    constexpr int COLS = 8 * NB;

    __shared__ float red[8][16][COLS];
    __shared__ float ss_part[NORM ? 8 : 1][16];
    __shared__ __align__(16) uint16_t nw_s[NORM ? K : 8];       // norm weights, staged once per CTA (not held in registers across the wait)

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int n0 = blockIdx.x * COLS;
    const int kbase = warp * KW + t * 8;

    const uint16_t* wrow[NB];
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) {
        int n = n0 + nb * 8 + g;
        n = n < N ? n : N - 1;
        wrow[nb] = W + (size_t)n * K + kbase;
    }
    const bool lo_ok = g < M, hi_ok = (g + 8) < M;
    const uint16_t* xlo = x + (size_t)(lo_ok ? g : 0) * K + kbase;
    const uint16_t* xhi = x + (size_t)(hi_ok ? g + 8 : 0) * K + kbase;

    float acc[NB][4];
#pragma unroll
    for (int nb = 0; nb < NB; ++nb)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[nb][i] = 0.f;

    const uint4 zero4 = make_uint4(0, 0, 0, 0);
    uint16_t r_old = 0;                  // EPI_RESID: this thread's element of the residual stream
    const int e_row = threadIdx.x / COLS, e_col = threadIdx.x % COLS;
#pragma unroll 1
    for (int c0 = 0; c0 < CH; c0 += BATCH) {
        uint4 wv[NB][BATCH];
#pragma unroll
        for (int c = 0; c < BATCH; ++c)
#pragma unroll
            for (int nb = 0; nb < NB; ++nb) wv[nb][c] = ldg16(wrow[nb] + (c0 + c) * 32);
        if (NORM && threadIdx.x < K / 8)          // immutable: ahead of the wait
            *reinterpret_cast<uint4*>(&nw_s[threadIdx.x * 8]) = ldg16(ex.nw + threadIdx.x * 8);
        if (c0 == 0) {
            if (ex.pf != nullptr && threadIdx.x == 0) l2_prefetch_slice(ex.pf, ex.pf_bytes, blockIdx.x, gridDim.x);
            pdl_wait();                   // the first batch of weight loads flies while the producer of x drains
            if (ex.trigger_early) pdl_trigger();
        }
        uint4 xl[BATCH], xh[BATCH];
#pragma unroll
        for (int c = 0; c < BATCH; ++c) {
            xl[c] = lo_ok ? __ldcg(reinterpret_cast<const uint4*>(xlo + (c0 + c) * 32)) : zero4;
            xh[c] = hi_ok ? __ldcg(reinterpret_cast<const uint4*>(xhi + (c0 + c) * 32)) : zero4;
        }
        if (EPI == EPI_RESID && c0 == 0 && threadIdx.x < 16 * COLS && e_row < M && n0 + e_col < N)
            r_old = __ldcg(static_cast<const uint16_t*>(out) + (size_t)e_row * N + n0 + e_col);
        if (NORM) {
            // rows g and g + 8: this thread's 32 values each, then lanes t = 0..3, then the eight warps
            float sl = 0.f, sh = 0.f;
#pragma unroll
            for (int c = 0; c < BATCH; ++c) {
                sl += sumsq8(xl[c]);
                sh += sumsq8(xh[c]);
            }
            sl += __shfl_xor_sync(0xffffffffu, sl, 1); sl += __shfl_xor_sync(0xffffffffu, sl, 2);
            sh += __shfl_xor_sync(0xffffffffu, sh, 1); sh += __shfl_xor_sync(0xffffffffu, sh, 2);
            if (t == 0) { ss_part[warp][g] = sl; ss_part[warp][g + 8] = sh; }
            __syncthreads();
            float al = 0.f, ah = 0.f;
#pragma unroll
            for (int w = 0; w < 8; ++w) { al += ss_part[w][g]; ah += ss_part[w][g + 8]; }
            const float il = rsqrt_acc(al * (1.0f / K) + kEps), ih = rsqrt_acc(ah * (1.0f / K) + kEps);
#pragma unroll
            for (int c = 0; c < BATCH; ++c) {
                const uint4 nwv = *reinterpret_cast<const uint4*>(&nw_s[kbase + c * 32]);     // staged before the barrier above
                xl[c] = norm8(xl[c], il, nwv);
                xh[c] = norm8(xh[c], ih, nwv);
            }
        }
#pragma unroll
        for (int c = 0; c < BATCH; ++c)
#pragma unroll
            for (int nb = 0; nb < NB; ++nb) {
                // the 8 values a thread holds are k = 8t..8t+7 of the chunk for BOTH operands, so
                // using {0,1|2,3} and {4,5|6,7} as the two k16 steps pairs equal k on both sides
                mma16816(acc[nb], xl[c].x, xh[c].x, xl[c].y, xh[c].y, wv[nb][c].x, wv[nb][c].y);
                mma16816(acc[nb], xl[c].z, xh[c].z, xl[c].w, xh[c].w, wv[nb][c].z, wv[nb][c].w);
            }
    }
    if (!ex.trigger_early) pdl_trigger();          // all loads are done: the successor may start fetching its weights
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) {
        red[warp][g][nb * 8 + 2 * t] = acc[nb][0];
        red[warp][g][nb * 8 + 2 * t + 1] = acc[nb][1];
        red[warp][g + 8][nb * 8 + 2 * t] = acc[nb][2];
        red[warp][g + 8][nb * 8 + 2 * t + 1] = acc[nb][3];
    }
    __syncthreads();

    if (EPI == EPI_RESID) {
        // thread = (row, column) of the CTA's 16 x COLS outputs; whole warps take part in the shuffles
        if (threadIdx.x < 16 * COLS) {
            float s = 0.f;
#pragma unroll
            for (int w = 0; w < 8; ++w) s += red[w][e_row][e_col];
            if (e_row < M && n0 + e_col < N)
                static_cast<uint16_t*>(out)[(size_t)e_row * N + n0 + e_col] = f2bf(bf2f(r_old) + bfround(s));
        }
    } else if (EPI == EPI_SWIGLU) {
        uint16_t* o = static_cast<uint16_t*>(out);
        const int ldo = N >> 1;
        for (int idx = threadIdx.x; idx < 16 * (COLS / 2); idx += 256) {
            const int row = idx / (COLS / 2), f = idx % (COLS / 2);
            if (row >= M || n0 + 2 * f + 1 >= N) continue;
            float gs = 0.f, us = 0.f;
#pragma unroll
            for (int w = 0; w < 8; ++w) { gs += red[w][row][2 * f]; us += red[w][row][2 * f + 1]; }
            o[(size_t)row * ldo + (n0 >> 1) + f] = swiglu_bf16(gs, us);
        }
    } else {
        __shared__ float vals[16][COLS];
        for (int idx = threadIdx.x; idx < 16 * COLS; idx += 256) {
            const int row = idx / COLS, col = idx % COLS;
            float s = 0.f;
#pragma unroll
            for (int w = 0; w < 8; ++w) s += red[w][row][col];
            if (EPI == EPI_PLAIN) {
                if (row < M && n0 + col < N)
                    static_cast<uint16_t*>(out)[(size_t)row * N + n0 + col] = f2bf(s);
            } else {
                vals[row][col] = s;
                if (logits != nullptr && row < M && n0 + col < N)
                    logits[(size_t)row * N + n0 + col] = s;
            }
        }
        if (EPI == EPI_ARGMAX) {
            __syncthreads();
            if (threadIdx.x < M) {
                const int row = threadIdx.x;
                float bv = -INFINITY;
                int bi = 0x7fffffff;
                for (int col = 0; col < COLS; ++col) {
                    const int n = n0 + col;
                    if (n < N && better(vals[row][col], n, bv, bi)) { bv = vals[row][col]; bi = n; }
                }
                partials[(size_t)row * n_parts + blockIdx.x] = ArgMax{bv, bi};
            }
        }
    }
}

// ------------------------------------------------------------------------------------------------
// rows > 16: tiled form
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
    const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(s), "l"(gmem));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }
__device__ __forceinline__ void ldmatrix_x4(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3,
                                            const void* smem) {
    const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(s));
}

template <int BM, int BN, int WARPS_M, int NWARPS, int STAGES, int EPI>
__global__ void __launch_bounds__(NWARPS * 32)
gemm_tiled_kernel(const uint16_t* __restrict__ x, const uint16_t* __restrict__ W, void* __restrict__ out,
                  int M, int N, int K, ArgMax* __restrict__ partials, float* __restrict__ logits,
                  int n_parts) {
    constexpr int BK = 64;
    constexpr int NT_THREADS = NWARPS * 32;
    constexpr int WARPS_N = NWARPS / WARPS_M;
    constexpr int WM = BM / WARPS_M, WN = BN / WARPS_N;
    constexpr int MT = WM / 16, NT = WN / 8;
    static_assert(WM % 16 == 0 && WN % 16 == 0, "warp tile");

    extern __shared__ __align__(128) uint16_t smem_raw[];
    uint16_t* As = smem_raw;                         // [STAGES][BM][64]
    uint16_t* Bs = smem_raw + STAGES * BM * BK;      // [STAGES][BN][64]

    pdl_wait();
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const int m0 = blockIdx.x * BM, n0 = blockIdx.y * BN;
    const int wm0 = (warp % WARPS_M) * WM, wn0 = (warp / WARPS_M) * WN;
    const int KT = K / BK;

    auto load_stage = [&](int s, int kt) {
        uint16_t* a = As + s * BM * BK;
        uint16_t* b = Bs + s * BN * BK;
        for (int i = tid; i < BM * 8; i += NT_THREADS) {
            const int r = i >> 3, c = i & 7;
            int gr = m0 + r;
            gr = gr < M ? gr : M - 1;
            cp_async16(a + r * BK + ((c ^ (r & 7)) << 3), x + (size_t)gr * K + kt * BK + c * 8);
        }
        for (int i = tid; i < BN * 8; i += NT_THREADS) {
            const int r = i >> 3, c = i & 7;
            int gr = n0 + r;
            gr = gr < N ? gr : N - 1;
            cp_async16(b + r * BK + ((c ^ (r & 7)) << 3), W + (size_t)gr * K + kt * BK + c * 8);
        }
    };

    float acc[MT][NT][4];
#pragma unroll
    for (int i = 0; i < MT; ++i)
#pragma unroll
        for (int j = 0; j < NT; ++j)
#pragma unroll
            for (int k = 0; k < 4; ++k) acc[i][j][k] = 0.f;

#pragma unroll
    for (int s = 0; s < STAGES - 1; ++s) {
        if (s < KT) load_stage(s, s);
        cp_async_commit();
    }

    for (int kt = 0; kt < KT; ++kt) {
        cp_async_wait<STAGES - 2>();
        __syncthreads();
        {
            const int nk = kt + STAGES - 1;
            if (nk < KT) load_stage(nk % STAGES, nk);
            cp_async_commit();
        }
        const uint16_t* a = As + (kt % STAGES) * BM * BK;
        const uint16_t* b = Bs + (kt % STAGES) * BN * BK;
#pragma unroll
        for (int kk = 0; kk < BK / 16; ++kk) {
            uint32_t af[MT][4];
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
                const int row = wm0 + mt * 16 + (lane & 15);
                const int chunk = kk * 2 + (lane >> 4);
                ldmatrix_x4(af[mt][0], af[mt][1], af[mt][2], af[mt][3],
                            a + row * BK + ((chunk ^ (row & 7)) << 3));
            }
            uint32_t bfr[NT][2];
#pragma unroll
            for (int np = 0; np < NT / 2; ++np) {
                const int row = wn0 + np * 16 + (lane & 7) + ((lane >> 4) << 3);
                const int chunk = kk * 2 + ((lane >> 3) & 1);
                ldmatrix_x4(bfr[2 * np][0], bfr[2 * np][1], bfr[2 * np + 1][0], bfr[2 * np + 1][1],
                            b + row * BK + ((chunk ^ (row & 7)) << 3));
            }
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                for (int nt = 0; nt < NT; ++nt)
                    mma16816(acc[mt][nt], af[mt][0], af[mt][1], af[mt][2], af[mt][3], bfr[nt][0],
                             bfr[nt][1]);
        }
    }
    cp_async_wait<0>();

    if (EPI == EPI_PLAIN) {
        uint16_t* o = static_cast<uint16_t*>(out);
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                const int col = n0 + wn0 + nt * 8 + 2 * t;
                if (col >= N) continue;
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const int row = m0 + wm0 + mt * 16 + g + h * 8;
                    if (row < M)
                        *reinterpret_cast<uint32_t*>(o + (size_t)row * N + col) =
                            pack_bf2(acc[mt][nt][2 * h], acc[mt][nt][2 * h + 1]);
                }
            }
    } else if (EPI == EPI_SWIGLU) {
        uint16_t* o = static_cast<uint16_t*>(out);
        const int ldo = N >> 1;
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                const int col = n0 + wn0 + nt * 8 + 2 * t;
                if (col >= N) continue;
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const int row = m0 + wm0 + mt * 16 + g + h * 8;
                    if (row < M)
                        o[(size_t)row * ldo + (col >> 1)] =
                            swiglu_bf16(acc[mt][nt][2 * h], acc[mt][nt][2 * h + 1]);
                }
            }
    } else {
        __shared__ ArgMax best[WARPS_N][BM];
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int rloc = wm0 + mt * 16 + g + h * 8;
                const int row = m0 + rloc;
                float bv = -INFINITY;
                int bi = 0x7fffffff;
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    const int col = n0 + wn0 + nt * 8 + 2 * t;
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        const float v = acc[mt][nt][2 * h + e];
                        if (col + e < N && better(v, col + e, bv, bi)) { bv = v; bi = col + e; }
                    }
                    if (logits != nullptr && row < M && col < N)
                        *reinterpret_cast<float2*>(logits + (size_t)row * N + col) =
                            make_float2(acc[mt][nt][2 * h], acc[mt][nt][2 * h + 1]);
                }
#pragma unroll
                for (int o = 1; o <= 2; o <<= 1) {
                    const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
                    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
                    if (better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
                }
                if (t == 0) best[warp / WARPS_M][rloc] = ArgMax{bv, bi};
            }
        __syncthreads();
        for (int r = tid; r < BM; r += NT_THREADS) {
            if (m0 + r >= M) continue;
            ArgMax b = best[0][r];
#pragma unroll
            for (int w = 1; w < WARPS_N; ++w)
                if (better(best[w][r].v, best[w][r].i, b.v, b.i)) b = best[w][r];
            partials[(size_t)(m0 + r) * n_parts + blockIdx.y] = b;
        }
    }
}

// ------------------------------------------------------------------------------------------------
// second stage of the argmax: one CTA per row scans that row's partials
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
argmax_final_kernel(const ArgMax* __restrict__ partials, int n_parts, int* __restrict__ tokens,
                    float* __restrict__ top_logit) {
    pdl_wait();
    pdl_trigger();
    const int row = blockIdx.x;
    const ArgMax* p = partials + (size_t)row * n_parts;
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = threadIdx.x; i < n_parts; i += 256) {
        const ArgMax c = p[i];
        if (better(c.v, c.i, bv, bi)) { bv = c.v; bi = c.i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
    }
    __shared__ ArgMax sm[8];
    if ((threadIdx.x & 31) == 0) sm[threadIdx.x >> 5] = ArgMax{bv, bi};
    __syncthreads();
    if (threadIdx.x == 0) {
        ArgMax b = sm[0];
        for (int w = 1; w < 8; ++w)
            if (better(sm[w].v, sm[w].i, b.v, b.i)) b = sm[w];
        tokens[row] = b.i;
        if (top_logit != nullptr) top_logit[row] = b.v;
    }
}

__global__ void pack_gate_up_kernel(const uint4* __restrict__ gate, const uint4* __restrict__ up,
                                    uint4* __restrict__ out) {
    // one 16-byte chunk per thread; 128 chunks per 1024-wide row
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t total = (size_t)kFF * 128;
    if (i >= total) return;
    const size_t f = i >> 7, c = i & 127;
    out[((2 * f) << 7) + c] = gate[i];
    out[((2 * f + 1) << 7) + c] = up[i];
}

// ------------------------------------------------------------------------------------------------
// host-side selection
// ------------------------------------------------------------------------------------------------
// A weight-streaming kernel lets its successor start right after its own wait: the successor's weight
// loads then overlap this kernel's arithmetic and tail (0.79 -> 0.75 ms per 1-lane step, 0.97 -> 0.92 ms
// at 16 lanes), and still only one successor is resident.  Q35_TRIG=0: after its arithmetic.
static int trigger_early() {
    static int mode = -1;
    if (mode < 0) {
        const char* env = std::getenv("Q35_TRIG");
        mode = (env != nullptr && env[0] == '0') ? 0 : 1;
    }
    return mode;
}

template <int K, int NB, int EPI, bool NORM = false>
static cudaError_t run_gemv(const uint16_t* x, const uint16_t* W, void* out, int M, int N,
                            ArgMax* partials, float* logits, int n_parts, cudaStream_t st,
                            const uint16_t* nw = nullptr, const void* pf = nullptr, size_t pf_bytes = 0) {
    const int grid = (N + 8 * NB - 1) / (8 * NB);
    const GemvExtra ex{nw, pf, (unsigned long long)pf_bytes, trigger_early()};
    return launch_k(gemv_rows_kernel<K, NB, EPI, NORM>, dim3(grid), dim3(256), 0, st, x, W, out, M, N, partials,
                    logits, n_parts, ex);
}

template <int BM, int BN, int WARPS_M, int NWARPS, int STAGES, int EPI>
static cudaError_t run_tiled(const uint16_t* x, const uint16_t* W, void* out, int M, int N, int K,
                             ArgMax* partials, float* logits, int n_parts, cudaStream_t st) {
    constexpr size_t smem = (size_t)STAGES * (BM + BN) * 64 * sizeof(uint16_t);
    static bool attr_done[kMaxDevices] = {false};   // per instantiation and device
    auto kern = gemm_tiled_kernel<BM, BN, WARPS_M, NWARPS, STAGES, EPI>;
    cudaError_t e = opt_in_smem(kern, smem, attr_done);
    if (e != cudaSuccess) return e;
    dim3 grid((M + BM - 1) / BM, (N + BN - 1) / BN);
    return launch_k(kern, grid, dim3(NWARPS * 32), smem, st, x, W, out, M, N, K, partials, logits, n_parts);
}

// tile choice of the tiled form: the largest tile whose grid still covers the SMs
struct TileChoice { int bm, bn; };
static TileChoice choose_tile(int M, int N) {
    auto ctas = [&](int bm, int bn) { return ((M + bm - 1) / bm) * ((N + bn - 1) / bn); };
    const int sms = sm_count();
    if (M > 64 && ctas(128, 128) >= sms) return {128, 128};
    if (M > 32 && ctas(64, 128) >= sms) return {64, 128};
    if (ctas(32, 128) >= sms || N > 2048) return {32, 128};
    if (M > 32 && ctas(64, 32) >= sms) return {64, 32};
    return {32, 32};
}

// The head of <= 16 rows runs on the tensor-memory kernels too (the form with the table as the M operand):
// it streams the 508 MB table at 6.1 TB/s against 3.7 TB/s for the GEMV form (83 vs 138 us at 16 rows), and
// a decode step and a verify body of any width then take their logits from tcgen05 accumulators.
// Q35_HEAD_TC=0 keeps the GEMV form.
static bool head_tc_few_rows() {
    static int mode = -1;
    if (mode < 0) {
        const char* env = std::getenv("Q35_HEAD_TC");
        mode = (env != nullptr && env[0] == '0') ? 0 : 1;
    }
    return mode == 1;
}

int linear_argmax_parts(int rows, int N) {
    if (rows <= 16 && !(head_tc_few_rows() && N >= 128))
        return (N + 31) / 32;                      // K = 1024 -> NB = 4 -> 32 weight rows per CTA
    return (N + 127) / 128;                        // argmax always runs BN = 128 tiles
}

template <int EPI>
static cudaError_t dispatch(const uint16_t* x, const uint16_t* W, void* out, int M, int N, int K,
                            ArgMax* partials, float* logits, int n_parts, cudaStream_t st) {
    if (M <= 16) {
        if (K == 1024) return run_gemv<1024, 4, EPI>(x, W, out, M, N, partials, logits, n_parts, st);
        if (EPI == EPI_PLAIN) {
            if (K == 2048) return run_gemv<2048, 1, EPI_PLAIN>(x, W, out, M, N, partials, logits, n_parts, st);
            if (K == 3584) return run_gemv<3584, 1, EPI_PLAIN>(x, W, out, M, N, partials, logits, n_parts, st);
        }
        return cudaErrorInvalidValue;
    }
    TileChoice tc = choose_tile(M, N);
    if (EPI == EPI_ARGMAX) tc.bn = 128, tc.bm = (M > 64 ? 128 : (M > 32 ? 64 : 32));
    if (tc.bn == 128) {
        if (tc.bm == 128) return run_tiled<128, 128, 2, 8, 3, EPI>(x, W, out, M, N, K, partials, logits, n_parts, st);
        if (tc.bm == 64) return run_tiled<64, 128, 2, 8, 4, EPI>(x, W, out, M, N, K, partials, logits, n_parts, st);
        return run_tiled<32, 128, 1, 8, 4, EPI>(x, W, out, M, N, K, partials, logits, n_parts, st);
    }
    if (EPI == EPI_PLAIN) {
        if (tc.bm == 64) return run_tiled<64, 32, 4, 8, 4, EPI_PLAIN>(x, W, out, M, N, K, partials, logits, n_parts, st);
        return run_tiled<32, 32, 2, 4, 4, EPI_PLAIN>(x, W, out, M, N, K, partials, logits, n_parts, st);
    }
    return run_tiled<32, 128, 1, 8, 4, EPI>(x, W, out, M, N, K, partials, logits, n_parts, st);
}

// which kernel launch_linear picks for a shape (the same conditions, in the same order)
const char* linear_route(int rows, int N, int K, int epi) {
    if (rows <= 0 || N <= 0 || (N & 7) || (K != 1024 && K != 2048 && K != 3584)) return "unsupported";
    if (linear_tc_eligible(rows, N, K) || (epi == EPI_ARGMAX && head_tc_few_rows() && N >= 128 && K % 64 == 0)) {
        if (epi == EPI_PLAIN && linear_tc_splits(rows, N, K, kSplitMaxRows) > 1) return "gemm_tc_kernel<128,4> split-K + add_norm_split_kernel";
        return linear_tc_route(rows, N, epi);
    }
    if (rows <= 16) return "gemv_rows_kernel";
    return "gemm_tiled_kernel (mma.sync)";
}

cudaError_t launch_linear(const uint16_t* x, const uint16_t* W, void* out, int rows, int N, int K,
                          int epi, ArgMax* partials, float* logits, int* n_parts_out, cudaStream_t st,
                          int* status) {
    if (rows <= 0 || N <= 0 || (N & 7) || (K != 1024 && K != 2048 && K != 3584))
        return cudaErrorInvalidValue;
    int n_parts = 0;
    if (epi == EPI_ARGMAX) {
        n_parts = linear_argmax_parts(rows, N);
        if (n_parts_out) *n_parts_out = n_parts;
    }
    if (linear_tc_eligible(rows, N, K) || (epi == EPI_ARGMAX && head_tc_few_rows() && N >= 128 && K % 64 == 0))
        return launch_linear_tc(x, W, out, rows, N, K, epi, partials, logits, n_parts, status, st);
    switch (epi) {
        case EPI_PLAIN: return dispatch<EPI_PLAIN>(x, W, out, rows, N, K, partials, logits, n_parts, st);
        case EPI_SWIGLU: return dispatch<EPI_SWIGLU>(x, W, out, rows, N, K, partials, logits, n_parts, st);
        case EPI_ARGMAX: return dispatch<EPI_ARGMAX>(x, W, out, rows, N, K, partials, logits, n_parts, st);
    }
    return cudaErrorInvalidValue;
}

// ---- fused residual stream (few rows) ---------------------------------------------------------
// Producer: resid [rows][1024] += x [rows][K] . W[1024][K]^T in place.  Consumer: out = N(resid; nw) . W^T
// with the norm applied while the rows are staged (every CTA holds all rows, so it takes their sums of
// squares from its own registers).  Between them no add + norm kernel runs.  pf / pf_bytes: weights of a
// later kernel to pull into L2 (optional).
cudaError_t launch_linear_resid_rows(const uint16_t* x, const uint16_t* W, uint16_t* resid, int rows, int K,
                                     const void* pf, size_t pf_bytes, cudaStream_t st) {
    if (rows < 1 || rows > 16) return cudaErrorInvalidValue;
    if (K == 2048) return run_gemv<2048, 1, EPI_RESID>(x, W, resid, rows, kHidden, nullptr, nullptr, 0, st, nullptr, pf, pf_bytes);
    if (K == 3584) return run_gemv<3584, 1, EPI_RESID>(x, W, resid, rows, kHidden, nullptr, nullptr, 0, st, nullptr, pf, pf_bytes);
    return cudaErrorInvalidValue;
}
cudaError_t launch_linear_norm_rows(const uint16_t* resid, const uint16_t* nw, const uint16_t* W, void* out, int rows,
                                    int N, int epi, const void* pf, size_t pf_bytes, cudaStream_t st) {
    if (rows < 1 || rows > 16 || N <= 0 || (N & 7)) return cudaErrorInvalidValue;
    if (epi == EPI_PLAIN)
        return run_gemv<1024, 4, EPI_PLAIN, true>(resid, W, out, rows, N, nullptr, nullptr, 0, st, nw, pf, pf_bytes);
    if (epi == EPI_SWIGLU)
        return run_gemv<1024, 4, EPI_SWIGLU, true>(resid, W, out, rows, N, nullptr, nullptr, 0, st, nw, pf, pf_bytes);
    return cudaErrorInvalidValue;
}

cudaError_t launch_argmax_final(const ArgMax* partials, int n_parts, int rows, int* tokens,
                                float* top_logit, cudaStream_t st) {
    return launch_k(argmax_final_kernel, dim3(rows), dim3(256), 0, st, partials, n_parts, tokens, top_logit);
}

// ------------------------------------------------------------------------------------------------
// tied head + argmax with the partial-argmax scratch in a fixed device array (no allocation)
// ------------------------------------------------------------------------------------------------
// The two-stage argmax needs rows x ceil(vocab / 32) (value, index) partials between its kernels.
// Here they live in this file-scope array, so the call never allocates.  The array is part of the
// library image: every GPU that loads the library holds these 1 MiB until the process exits.
static __device__ __align__(256) ArgMax g_static_partials[kStaticHeadMaxRows * (kStaticHeadMaxVocab / 32)];

cudaError_t launch_lm_head_static(const uint16_t* x, const uint16_t* embed, int vocab, int rows,
                                  int* tokens, cudaStream_t st) {
    if (rows < 1 || rows > kStaticHeadMaxRows || vocab < 8 || vocab > kStaticHeadMaxVocab || (vocab & 7))
        return cudaErrorInvalidValue;
    // In host code `g_static_partials` is only a handle for the symbol, not a device address, so
    // the address each device gave the array is looked up once per device and remembered.
    static ArgMax* dev_ptr[64] = {nullptr};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
    if (dev_ptr[dev] == nullptr) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_static_partials);
        if (e != cudaSuccess) return e;
        dev_ptr[dev] = static_cast<ArgMax*>(p);
    }
    ArgMax* partials = dev_ptr[dev];
    const int n_parts = (vocab + 31) / 32;
    // every partial that the second kernel reads is written by the first one in this same call,
    // so nothing left over from an earlier call needs clearing
    e = run_gemv<1024, 4, EPI_ARGMAX>(x, embed, nullptr, rows, vocab, partials, nullptr, n_parts, st);
    if (e != cudaSuccess) return e;
    return launch_k(argmax_final_kernel, dim3(rows), dim3(256), 0, st, static_cast<const ArgMax*>(partials), n_parts, tokens,
                    static_cast<float*>(nullptr));
}

cudaError_t launch_pack_gate_up(const uint16_t* gate, const uint16_t* up, uint16_t* out, cudaStream_t st) {
    const size_t total = (size_t)kFF * 128;
    pack_gate_up_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>(
        reinterpret_cast<const uint4*>(gate), reinterpret_cast<const uint4*>(up),
        reinterpret_cast<uint4*>(out));
    return cudaGetLastError();
}

}  // namespace q35
