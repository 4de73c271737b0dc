// GatedDeltaNet step: causal conv1d roll + SiLU, gates, q/k L2 norm, the f32 delta-rule update of
// the 128x128 per-head state, and the gated RMSNorm, in ONE kernel per layer.
//
// Persistent CTAs (two per SM; each keeps one head and strides over lanes) walk the (lane, head)
// items of a layer.  Everything the NEXT item needs from HBM - its 64 KiB head state, its q/k/v
// rows, conv window rows and z row - is fetched into shared memory by bulk async copies
// (cp.async.bulk, completion on one mbarrier) while the current item is updated, so every SM keeps
// state loads in flight all the time and no global-load latency sits on an item's critical path.  The current tile lives in registers (thread = 16 rows x 4 columns): both reductions of the
// update (r = S^T k and o = S^T q) run on the register copy with a cross-warp shared-memory reduce,
// and the new state is written back exactly once with 16-byte stores.  This is the HBM term that
// dominates the step at high lane counts (2 x 1 MiB per layer per lane).
// The mbarrier wait is bounded (about one second of polling): on expiry the kernel raises the
// status word it was given and returns.
//
// Replaces gdn_conv / gdn_gates / gdn_rec / gdn_gated_norm (engine/kernels.h:398-460,682);
// arithmetic follows speccheck/specimpl.py:252-305 as executed.
#include <cstdlib>

#include "q35_common.cuh"

namespace q35 {

constexpr int kOffZ = 6144, kOffB = 8192, kOffA = 8208;
constexpr uint32_t kTileBytes = kDk * kDv * sizeof(float);   // 65,536

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

// Poll the barrier's phase; give up after ~1 s.  Returns false on expiry.
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity) {
    const unsigned long long t0 = global_ns();
    for (;;) {
        uint32_t ok;
        asm volatile(
            "{\n .reg .pred p;\n mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n"
            " selp.u32 %0, 1, 0, p;\n}\n"
            : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
        if (ok) return true;
        if (global_ns() - t0 > 1000000000ull) return false;
        __nanosleep(20);
    }
}

__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n"
        ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

constexpr int kInRows = 13;                                   // q, k, v raw | 3x3 window | z, 128 bf16 each
constexpr uint32_t kInBytes = kInRows * 128 * sizeof(uint16_t);
constexpr uint32_t kFetchBytes = kTileBytes + kInBytes;
constexpr size_t kGdnSmemBytes = kTileBytes + kInBytes;

// One thread: everything item (lane_id, h) needs from HBM for its first token, as bulk copies that
// complete on one mbarrier: the 64 KiB state tile and thirteen 256-byte rows of small inputs.
// Two parts: the state tile and conv window (written by this layer's previous step only) and the
// rows of this step's projection; the first may be issued before the projection kernel has ended.
__device__ __forceinline__ void item_fetch_state(const GdnParams& p, int lane_id, int h, uint32_t tile_addr,
                                                 uint32_t in_addr, uint32_t bar) {
    const int sel = p.sel != nullptr ? p.sel[lane_id] : 0;
    const float* S = pick_buf(p.S, sel) + ((size_t)lane_id * kGdnHeads + h) * (kDk * kDv);
    const uint16_t* win = pick_buf(p.win, sel) + (size_t)lane_id * 3 * kConvCh;
    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(kFetchBytes) : "memory");
    bulk_g2s(tile_addr, S, kTileBytes, bar);
#pragma unroll
    for (int kind = 0; kind < 3; ++kind)
#pragma unroll
        for (int j = 0; j < 3; ++j)
            bulk_g2s(in_addr + (3 + j * 3 + kind) * 256, win + j * kConvCh + kind * 2048 + h * 128, 256, bar);
}
__device__ __forceinline__ void item_fetch_rows(const GdnParams& p, int lane_id, int h, uint32_t in_addr,
                                                uint32_t bar) {
    const uint16_t* pr = p.proj + (size_t)lane_id * p.T * kGdnProjN;
#pragma unroll
    for (int kind = 0; kind < 3; ++kind) bulk_g2s(in_addr + kind * 256, pr + kind * 2048 + h * 128, 256, bar);
    bulk_g2s(in_addr + 12 * 256, pr + kOffZ + h * 128, 256, bar);
}
__device__ __forceinline__ void item_fetch(const GdnParams& p, int lane_id, int h, uint32_t tile_addr,
                                           uint32_t in_addr, uint32_t bar) {
    item_fetch_state(p, lane_id, h, tile_addr, in_addr, bar);
    item_fetch_rows(p, lane_id, h, in_addr, bar);
}

__global__ void __launch_bounds__(256, 2) gdn_step_kernel(GdnParams p) {
    extern __shared__ __align__(128) unsigned char dyn_smem[];
    float* tile = reinterpret_cast<float*>(dyn_smem);                          // 128x128 f32 head tile
    uint16_t* in_s = reinterpret_cast<uint16_t*>(dyn_smem + kTileBytes);       // [13][128] bf16
    __shared__ __align__(8) unsigned long long bar_storage;
    __shared__ float q_s[128], k_s[128], v_s[128];
    __shared__ __align__(16) float red_r[8][128];
    __shared__ __align__(16) float red_o[8][128];
    __shared__ float ssum[4][2];
    __shared__ float scal_s[2];

    const int tid = threadIdx.x, warp = tid >> 5, ln = tid & 31;
    // the grid is a multiple of 16, so a CTA keeps one head and strides over lanes
    const int h = blockIdx.x % kGdnHeads;
    const int lane_stride = gridDim.x / kGdnHeads;
    const uint32_t bar = smem_u32(&bar_storage);
    const uint32_t tile_addr = smem_u32(tile), in_addr = smem_u32(in_s);
    float nb_raw = 0.f, na_raw = 0.f;          // thread 0: gate inputs of the item being fetched
    {
        // the first state tile is on its way before the projection kernel ahead of this one has ended
        const int l0 = blockIdx.x / kGdnHeads;
        if (tid == 0) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;\n" ::"r"(bar) : "memory");
            asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
            if (l0 < p.lanes) item_fetch_state(p, l0, h, tile_addr, in_addr, bar);
        }
        pdl_wait();
        __syncthreads();
        if (tid == 0 && l0 < p.lanes) {
            item_fetch_rows(p, l0, h, in_addr, bar);
            const uint16_t* pr0 = p.proj + (size_t)l0 * p.T * kGdnProjN;
            nb_raw = bf2f(pr0[kOffB + h]);
            na_raw = bf2f(pr0[kOffA + h]);
        }
    }

    // per-CTA constants of head h
    const float negA = -expf(bf2f(p.A_log[h]));
    const float dtb = bf2f(p.dt_bias[h]);
    const float q_scale = 0.08838834764831845f;   // 128^-1/2
    float tap[3][4];
    int ch[3] = {0, 0, 0};
    if (tid < 128) {
#pragma unroll
        for (int kind = 0; kind < 3; ++kind) {
            ch[kind] = kind * 2048 + h * 128 + tid;
            const uint2 tw = *reinterpret_cast<const uint2*>(p.conv_w + (size_t)ch[kind] * 4);
            tap[kind][0] = lo_bf(tw.x); tap[kind][1] = hi_bf(tw.x);
            tap[kind][2] = lo_bf(tw.y); tap[kind][3] = hi_bf(tw.y);
        }
    }
    float nw4[4] = {0.f, 0.f, 0.f, 0.f};
    if (warp == 0) {
        const uint2 nv = *reinterpret_cast<const uint2*>(p.norm_w + 4 * ln);
        nw4[0] = lo_bf(nv.x); nw4[1] = hi_bf(nv.x); nw4[2] = lo_bf(nv.y); nw4[3] = hi_bf(nv.y);
    }

    uint32_t phase = 0;
    for (int lane_id = blockIdx.x / kGdnHeads; lane_id < p.lanes; lane_id += lane_stride) {
        const int sel = p.sel != nullptr ? p.sel[lane_id] : 0;
        const size_t s_off = ((size_t)lane_id * kGdnHeads + h) * (kDk * kDv);
        const size_t w_off = (size_t)lane_id * 3 * kConvCh;
        float* S_live = pick_buf(p.S, sel) + s_off;
        uint16_t* win_live = pick_buf(p.win, sel) + w_off;

        // ---- prefetched tile and inputs: shared memory -> registers ------------------------------
        if (!mbar_wait_bounded(bar, phase)) {
            if (tid == 0 && p.status != nullptr) atomicExch(p.status, 1);
            return;
        }
        phase ^= 1;
        float4 s[16];
        {
            const float4* Sp = reinterpret_cast<const float4*>(tile);
#pragma unroll
            for (int r = 0; r < 16; ++r) s[r] = Sp[(warp * 16 + r) * 32 + ln];
        }
        float raw0[3] = {0.f, 0.f, 0.f}, win[3][3];
        uint2 z4 = make_uint2(0, 0);
        if (warp == 0) z4 = *reinterpret_cast<const uint2*>(in_s + 12 * 128 + 4 * ln);
        if (tid < 128) {
#pragma unroll
            for (int kind = 0; kind < 3; ++kind) {
                raw0[kind] = bf2f(in_s[kind * 128 + tid]);
#pragma unroll
                for (int j = 0; j < 3; ++j) win[kind][j] = bf2f(in_s[(3 + j * 3 + kind) * 128 + tid]);
            }
        }
        if (tid == 0) { scal_s[0] = nb_raw; scal_s[1] = na_raw; }
        __syncthreads();                   // every thread has its copy: the buffers are free again
        if (tid == 0) {
            const int nxt = lane_id + lane_stride;
            if (nxt < p.lanes) {
                item_fetch(p, nxt, h, tile_addr, in_addr, bar);
                const uint16_t* prn = p.proj + (size_t)nxt * p.T * kGdnProjN;
                nb_raw = bf2f(prn[kOffB + h]);
                na_raw = bf2f(prn[kOffA + h]);
            } else {
                pdl_trigger();             // last item of this CTA: the next kernel may start its weight loads
            }
        }

        for (int t = 0; t < p.T; ++t) {
            const size_t row = (size_t)lane_id * p.T + t;
            const uint16_t* pr = p.proj + row * kGdnProjN;

            // ---- conv (f32 taps in ascending order, one bf16 rounding) + SiLU in bf16 ---------
            if (tid < 128) {
                float u[3];
#pragma unroll
                for (int kind = 0; kind < 3; ++kind) {
                    const float raw = (t == 0) ? raw0[kind] : bf2f(pr[ch[kind]]);
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

            // ---- gates and norms (every thread computes the same scalars) ---------------------
            const float qinv = rsqrt_acc(ssum[0][0] + ssum[1][0] + ssum[2][0] + ssum[3][0] + 1e-6f);
            const float kinv = rsqrt_acc(ssum[0][1] + ssum[1][1] + ssum[2][1] + ssum[3][1] + 1e-6f);
            const float b_raw = (t == 0) ? scal_s[0] : bf2f(pr[kOffB + h]);
            const float a_raw = (t == 0) ? scal_s[1] : bf2f(pr[kOffA + h]);
            const float beta = sigmoid_acc(b_raw);
            const float sp_in = a_raw + dtb;
            const float sp = sp_in > 20.0f ? sp_in : log1pf(expf(sp_in));
            const float gamma = expf(__fmul_rn(negA, sp));

            // ---- S <- gamma S ; r = S^T k ------------------------------------------------------
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

            // ---- dv = beta (v - r) ; S <- S + k (x) dv ; o = S^T q -----------------------------
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

            // ---- gated RMSNorm over the head's 128 outputs (f32 until the single bf16 cast) ----
            // warp 0 alone: a lane takes 4 columns, so the mean square needs no block barrier and the
            // other warps move on to their state stores / the next item
            if (warp == 0) {
                float4 o4 = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                for (int w = 0; w < 8; ++w) {
                    const float4 a = *reinterpret_cast<const float4*>(&red_o[w][4 * ln]);
                    o4.x += a.x; o4.y += a.y; o4.z += a.z; o4.w += a.w;
                }
                const float ms = warp_sum(o4.x * o4.x + o4.y * o4.y + o4.z * o4.z + o4.w * o4.w) * (1.0f / 128.0f);
                const float rinv = rsqrt_acc(ms + kEps);
                uint2 zr = z4;
                if (t > 0) zr = *reinterpret_cast<const uint2*>(pr + kOffZ + h * 128 + 4 * ln);
                const float zf[4] = {lo_bf(zr.x), hi_bf(zr.x), lo_bf(zr.y), hi_bf(zr.y)};
                const float of[4] = {o4.x, o4.y, o4.z, o4.w};
                float out[4];
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    float n = __fmul_rn(of[c], rinv);
                    n = __fmul_rn(nw4[c], n);
                    out[c] = __fmul_rn(n, silu_acc(zf[c]));
                }
                *reinterpret_cast<uint2*>(p.y + row * kValueDim + h * 128 + 4 * ln) =
                    make_uint2(pack_bf2(out[0], out[1]), pack_bf2(out[2], out[3]));
            }

            // ---- checkpoint after every non-final token of a speculative verify body -------------
            if (t < p.checkpoint) {
                int cb = sel + 1 + t;
                if (cb > p.checkpoint) cb -= p.checkpoint + 1;
                float4* Sc = reinterpret_cast<float4*>(pick_buf(p.S, cb) + s_off);
#pragma unroll
                for (int r = 0; r < 16; ++r) Sc[(warp * 16 + r) * 32 + ln] = s[r];
                if (tid < 128) {
                    uint16_t* wc = pick_buf(p.win, cb) + w_off;
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
}

cudaError_t launch_gdn_step(const GdnParams& p, cudaStream_t st) {
    if (p.lanes <= 0 || p.T <= 0 || p.lanes > 65535) return cudaErrorInvalidValue;
    if (p.checkpoint < 0 || p.checkpoint >= kStateBufs) return cudaErrorInvalidValue;
    if (p.checkpoint > 0) {
        if (p.T != p.checkpoint + 1) return cudaErrorInvalidValue;
        for (int b = 0; b <= p.checkpoint; ++b)
            if (p.S[b] == nullptr || p.win[b] == nullptr) return cudaErrorInvalidValue;
    }
    static int max_ctas = 0;
    if (max_ctas == 0) {
        int dev = 0, sms = 0;
        cudaError_t e = cudaGetDevice(&dev);
        if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        if (e == cudaSuccess)
            e = cudaFuncSetAttribute(gdn_step_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kGdnSmemBytes);
        if (e != cudaSuccess) return e;
        int per_sm = 2;
        if (const char* env = std::getenv("Q35_GDN_CTAS_PER_SM")) per_sm = env[0] == '1' ? 1 : 2;   // tuning knob
        max_ctas = (per_sm * sms / kGdnHeads) * kGdnHeads;  // two CTAs per SM, rounded down to whole lanes
        if (max_ctas < kGdnHeads) max_ctas = kGdnHeads;
    }
    const int items = p.lanes * kGdnHeads;
    const int grid = items < max_ctas ? items : max_ctas;
    return launch_k(gdn_step_kernel, dim3(grid), dim3(256), kGdnSmemBytes, st, p);
}

}  // namespace q35
