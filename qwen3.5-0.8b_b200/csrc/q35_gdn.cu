// GatedDeltaNet step: causal conv1d roll + SiLU, gates, q/k L2 norm, the f32 delta-rule update of
// the 128x128 per-head state, and the gated RMSNorm, in ONE kernel per layer.
//
// One CTA per (head, lane).  The 64 KiB head state is read from HBM exactly once into registers
// (thread = 16 rows x 4 columns, so a warp reads whole 512-byte state rows), both reductions of
// the update (r = S^T k and o = S^T q) run on the register copy with a cross-warp shared-memory
// reduce, and the new state is written back exactly once.  This is the HBM term that dominates
// the step at high lane counts (2 x 1 MiB per layer per lane).
//
// Replaces gdn_conv / gdn_gates / gdn_rec / gdn_gated_norm (engine/kernels.h:398-460,682);
// arithmetic follows speccheck/specimpl.py:252-305 as executed.
#include "q35_common.cuh"

namespace q35 {

constexpr int kOffZ = 6144, kOffB = 8192, kOffA = 8208;

__global__ void __launch_bounds__(256, 2) gdn_step_kernel(GdnParams p) {
    const int h = blockIdx.x, lane_id = blockIdx.y;
    const int tid = threadIdx.x, warp = tid >> 5, ln = tid & 31;

    __shared__ float q_s[128], k_s[128], v_s[128];
    __shared__ __align__(16) float red_r[8][128];
    __shared__ __align__(16) float red_o[8][128];
    __shared__ float ssum[4][2];
    __shared__ float osum[4];

    const int sel = p.sel != nullptr ? (p.sel[lane_id] & 1) : 0;
    const size_t s_off = ((size_t)lane_id * kGdnHeads + h) * (kDk * kDv);
    const size_t w_off = (size_t)lane_id * 3 * kConvCh;
    float* S_live = p.S[sel] + s_off;
    uint16_t* win_live = p.win[sel] + w_off;

    // ---- state tile -> registers (issued first so the loads fly under the conv) --------------
    float4 s[16];
    {
        const float4* Sp = reinterpret_cast<const float4*>(S_live);
#pragma unroll
        for (int r = 0; r < 16; ++r) s[r] = Sp[(warp * 16 + r) * 32 + ln];
    }

    const float negA = -expf(bf2f(p.A_log[h]));
    const float dtb = bf2f(p.dt_bias[h]);
    const float q_scale = 0.08838834764831845f;   // 128^-1/2

    // conv taps and window for this thread's three channels (q, k, v of column `tid`)
    float tap[3][4], win[3][3];
    int ch[3] = {0, 0, 0};
    float nw = 0.f;
    if (tid < 128) {
#pragma unroll
        for (int kind = 0; kind < 3; ++kind) {
            ch[kind] = kind * 2048 + h * 128 + tid;
            const uint2 tw = *reinterpret_cast<const uint2*>(p.conv_w + (size_t)ch[kind] * 4);
            tap[kind][0] = lo_bf(tw.x); tap[kind][1] = hi_bf(tw.x);
            tap[kind][2] = lo_bf(tw.y); tap[kind][3] = hi_bf(tw.y);
#pragma unroll
            for (int j = 0; j < 3; ++j) win[kind][j] = bf2f(win_live[j * kConvCh + ch[kind]]);
        }
        nw = bf2f(p.norm_w[tid]);
    }

    for (int t = 0; t < p.T; ++t) {
        const size_t row = (size_t)lane_id * p.T + t;
        const uint16_t* pr = p.proj + row * kGdnProjN;

        // ---- conv (f32 taps in ascending order, one bf16 rounding) + SiLU in bf16 -------------
        if (tid < 128) {
            float u[3];
#pragma unroll
            for (int kind = 0; kind < 3; ++kind) {
                const float raw = bf2f(pr[ch[kind]]);
                float acc = __fmul_rn(win[kind][0], tap[kind][0]);
                acc = __fadd_rn(acc, __fmul_rn(win[kind][1], tap[kind][1]));
                acc = __fadd_rn(acc, __fmul_rn(win[kind][2], tap[kind][2]));
                acc = __fadd_rn(acc, __fmul_rn(raw, tap[kind][3]));
                u[kind] = bfround(silu_acc(bfround(acc)));
                win[kind][0] = win[kind][1]; win[kind][1] = win[kind][2]; win[kind][2] = raw;
            }
            q_s[tid] = u[0]; k_s[tid] = u[1]; v_s[tid] = u[2];
            const float qq = warp_sum(u[0] * u[0]);
            const float kk = warp_sum(u[1] * u[1]);
            if (ln == 0) { ssum[warp][0] = qq; ssum[warp][1] = kk; }
        }
        __syncthreads();

        // ---- gates and norms (every thread computes the same scalars) -------------------------
        const float qinv = rsqrt_acc(ssum[0][0] + ssum[1][0] + ssum[2][0] + ssum[3][0] + 1e-6f);
        const float kinv = rsqrt_acc(ssum[0][1] + ssum[1][1] + ssum[2][1] + ssum[3][1] + 1e-6f);
        const float beta = sigmoid_acc(bf2f(pr[kOffB + h]));
        const float sp_in = bf2f(pr[kOffA + h]) + dtb;
        const float sp = sp_in > 20.0f ? sp_in : log1pf(expf(sp_in));
        const float gamma = expf(__fmul_rn(negA, sp));

        // ---- S <- gamma S ; r = S^T k ----------------------------------------------------------
        float4 pr4 = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int r = 0; r < 16; ++r) {
            const float kh = __fmul_rn(k_s[warp * 16 + r], kinv);
            s[r].x = __fmul_rn(s[r].x, gamma); s[r].y = __fmul_rn(s[r].y, gamma);
            s[r].z = __fmul_rn(s[r].z, gamma); s[r].w = __fmul_rn(s[r].w, gamma);
            pr4.x += s[r].x * kh; pr4.y += s[r].y * kh; pr4.z += s[r].z * kh; pr4.w += s[r].w * kh;
        }
        *reinterpret_cast<float4*>(&red_r[warp][4 * ln]) = pr4;
        __syncthreads();

        // ---- dv = beta (v - r) ; S <- S + k (x) dv ; o = S^T q ---------------------------------
        float4 rj = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int w = 0; w < 8; ++w) {
            const float4 a = *reinterpret_cast<const float4*>(&red_r[w][4 * ln]);
            rj.x += a.x; rj.y += a.y; rj.z += a.z; rj.w += a.w;
        }
        float4 dv;
        dv.x = __fmul_rn(beta, v_s[4 * ln + 0] - rj.x);
        dv.y = __fmul_rn(beta, v_s[4 * ln + 1] - rj.y);
        dv.z = __fmul_rn(beta, v_s[4 * ln + 2] - rj.z);
        dv.w = __fmul_rn(beta, v_s[4 * ln + 3] - rj.w);
        float4 po = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int r = 0; r < 16; ++r) {
            const float kh = __fmul_rn(k_s[warp * 16 + r], kinv);
            const float qh = __fmul_rn(__fmul_rn(q_s[warp * 16 + r], qinv), q_scale);
            s[r].x = __fadd_rn(s[r].x, __fmul_rn(kh, dv.x));
            s[r].y = __fadd_rn(s[r].y, __fmul_rn(kh, dv.y));
            s[r].z = __fadd_rn(s[r].z, __fmul_rn(kh, dv.z));
            s[r].w = __fadd_rn(s[r].w, __fmul_rn(kh, dv.w));
            po.x += s[r].x * qh; po.y += s[r].y * qh; po.z += s[r].z * qh; po.w += s[r].w * qh;
        }
        *reinterpret_cast<float4*>(&red_o[warp][4 * ln]) = po;
        __syncthreads();

        // ---- gated RMSNorm over the head's 128 outputs (f32 until the single bf16 cast) --------
        float o = 0.f;
        if (tid < 128) {
#pragma unroll
            for (int w = 0; w < 8; ++w) o += red_o[w][tid];
            const float oo = warp_sum(o * o);
            if (ln == 0) osum[warp] = oo;
        }
        __syncthreads();
        if (tid < 128) {
            const float ms = (osum[0] + osum[1] + osum[2] + osum[3]) * (1.0f / 128.0f);
            float n = __fmul_rn(o, rsqrt_acc(ms + kEps));
            n = __fmul_rn(nw, n);
            const float z = bf2f(pr[kOffZ + h * 128 + tid]);
            p.y[row * kValueDim + h * 128 + tid] = f2bf(__fmul_rn(n, silu_acc(z)));
        }

        // ---- checkpoint after the first of two tokens (speculative verify) ---------------------
        if (p.checkpoint && t == 0) {
            float4* Sc = reinterpret_cast<float4*>(p.S[sel ^ 1] + s_off);
#pragma unroll
            for (int r = 0; r < 16; ++r) Sc[(warp * 16 + r) * 32 + ln] = s[r];
            if (tid < 128) {
                uint16_t* wc = p.win[sel ^ 1] + w_off;
#pragma unroll
                for (int kind = 0; kind < 3; ++kind)
#pragma unroll
                    for (int j = 0; j < 3; ++j) wc[j * kConvCh + ch[kind]] = f2bf(win[kind][j]);
            }
        }
    }

    {
        float4* So = reinterpret_cast<float4*>(S_live);
#pragma unroll
        for (int r = 0; r < 16; ++r) So[(warp * 16 + r) * 32 + ln] = s[r];
    }
    if (tid < 128) {
#pragma unroll
        for (int kind = 0; kind < 3; ++kind)
#pragma unroll
            for (int j = 0; j < 3; ++j) win_live[j * kConvCh + ch[kind]] = f2bf(win[kind][j]);
    }
}

cudaError_t launch_gdn_step(const GdnParams& p, cudaStream_t st) {
    if (p.lanes <= 0 || p.T <= 0 || p.lanes > 65535) return cudaErrorInvalidValue;
    if (p.checkpoint && (p.T != 2 || p.S[1] == nullptr || p.win[1] == nullptr)) return cudaErrorInvalidValue;
    gdn_step_kernel<<<dim3(kGdnHeads, p.lanes), 256, 0, st>>>(p);
    return cudaGetLastError();
}

}  // namespace q35
