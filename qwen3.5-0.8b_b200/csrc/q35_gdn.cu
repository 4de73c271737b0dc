// GatedDeltaNet step: causal conv1d roll + SiLU, gates, q/k L2 norm, the f32 delta-rule update of
// the 128x128 per-head state, and the gated RMSNorm, in ONE kernel per layer.
//
// Persistent CTAs (two per SM; each keeps one head and strides over lanes) walk the (lane, head)
// items of a layer.  Everything the NEXT item needs from HBM - its 64 KiB head state, its q/k/v
// rows, conv window rows and z row - is fetched into shared memory by bulk async copies
// (one cp.async.bulk for the tile, one 3-D and one 4-D tensor copy for the small pieces, completion
// on one mbarrier) while the current item is updated, so every SM keeps
// state loads in flight all the time and no global-load latency sits on an item's critical path.
// The current tile lives in registers (thread = 16 rows x 4 columns): both reductions of the
// update (r = S^T k and o = S^T q) run on the register copy with a cross-warp shared-memory reduce,
// and the new state is written back exactly once with 16-byte stores.  This is the HBM term that
// dominates the step at high lane counts (2 x 1 MiB per layer per lane).
// What every warp must do per item is one chain (copy, conv, pass 1, pass 2, stores); everything
// else is given to warps that would otherwise idle in the conv stage (see the kernel's comment), so
// that the chain, not one overloaded warp, sets the pace and two CTAs per SM saturate HBM.
// The mbarrier wait is bounded (about one second of polling): on expiry the kernel raises the
// status word it was given and returns.
//
// Replaces gdn_conv / gdn_gates / gdn_rec / gdn_gated_norm (engine/kernels.h:398-460,682);
// arithmetic follows speccheck/specimpl.py:252-305 as executed.
#include <cuda.h>

#include <cstdlib>
#include <mutex>
#include <unordered_map>

#include "q35_common.cuh"
#include "q35_async.cuh"

namespace q35 {

constexpr int kOffZ = 6144, kOffB = 8192, kOffA = 8208;
constexpr uint32_t kTileBytes = kDk * kDv * sizeof(float);   // 65,536

constexpr int kInRows = 13;                                   // q, k, v raw | 3x3 window | z, 128 bf16 each
constexpr uint32_t kInBytes = kInRows * 128 * sizeof(uint16_t);
constexpr uint32_t kFetchBytes = kTileBytes + kInBytes;
constexpr size_t kGdnSmemBytes = kTileBytes + kInBytes;

// Everything item (lane_id, h) needs from HBM for its first token, as THREE copies that complete on
// one mbarrier (issuing a copy costs the issuing warp ~130 cycles, one after the other, on the chain
// every warp waits for): the 64 KiB state tile (bulk copy), the head's q | k | v | z pieces of the
// projection row (one 3-D tensor copy: 4 pieces of 128 values, 2048 apart), and the head's 3 x 3
// conv-window pieces (one 4-D tensor copy).  Shared-memory rows: 0..3 = q, k, v, z; 4 + 3 j + kind =
// window row j of kind.  `what` bit 0: the state tile and conv window (written by this layer's
// previous step only), bit 1: the projection pieces; the first may be issued before the projection
// kernel ahead of this one has ended.
__device__ __forceinline__ void item_fetch(const GdnParams& p, const CUtensorMap* pmap, const CUtensorMap* wmap0,
                                           const CUtensorMap* wmap1, const CUtensorMap* wmap2, int lane_id, int h,
                                           int what, uint32_t tile_addr, uint32_t in_addr, uint32_t bar) {
    const int sel = p.sel != nullptr ? p.sel[lane_id] : 0;
    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
    if (what & 1) {
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(kFetchBytes) : "memory");
        bulk_g2s(tile_addr, pick_buf(p.S, sel) + ((size_t)lane_id * kGdnHeads + h) * (kDk * kDv), kTileBytes, bar);
        const CUtensorMap* wm = sel == 0 ? wmap0 : (sel == 1 ? wmap1 : wmap2);
        asm volatile(
            "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];\n"
            ::"r"(in_addr + 4 * 256), "l"(reinterpret_cast<uint64_t>(wm)), "r"(bar), "r"(h * 128), "r"(0), "r"(0), "r"(lane_id) : "memory");
    }
    if (what & 2)
        asm volatile(
            "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];\n"
            ::"r"(in_addr), "l"(reinterpret_cast<uint64_t>(pmap)), "r"(bar), "r"(h * 128), "r"(0), "r"(lane_id * p.T) : "memory");
}

// conv taps stay packed as two bf16 pairs; f32 taps in ascending order, one bf16 rounding, SiLU in bf16
__device__ __forceinline__ float conv_silu(float (&w)[3], float raw, uint2 tap) {
    float acc = __fmul_rn(w[0], lo_bf(tap.x));
    acc = __fadd_rn(acc, __fmul_rn(w[1], hi_bf(tap.x)));
    acc = __fadd_rn(acc, __fmul_rn(w[2], lo_bf(tap.y)));
    acc = __fadd_rn(acc, __fmul_rn(raw, hi_bf(tap.y)));
    w[0] = w[1]; w[1] = w[2]; w[2] = raw;
    return bfround(silu_acc(bfround(acc)));
}

// Warp roles.  Warps 0-3 (thread = channel c): conv of q and v.  Warps 4-7 (thread = channel /
// column c): conv of k, the gated RMSNorm of column c, and - warp 4 - the fetch of the next item.
// The gated norm of an item's last token is DEFERRED: it runs after the next item's tile has been
// copied to registers, in the shadow of that item's conv (which warps 0-3 carry the longer half
// of), so neither the norm nor the fetch sits on the chain conv -> pass 1 -> pass 2 -> stores that
// every warp walks.
__global__ void __launch_bounds__(256, 2)
gdn_step_kernel(GdnParams p, const __grid_constant__ CUtensorMap pmap, const __grid_constant__ CUtensorMap wmap0,
                const __grid_constant__ CUtensorMap wmap1, const __grid_constant__ CUtensorMap wmap2) {
    extern __shared__ __align__(128) unsigned char dyn_smem[];
    float* tile = reinterpret_cast<float*>(dyn_smem);                          // 128x128 f32 head tile
    uint16_t* in_s = reinterpret_cast<uint16_t*>(dyn_smem + kTileBytes);       // [13][128] bf16
    __shared__ __align__(8) unsigned long long bar_storage;
    __shared__ float q_s[128], k_s[128], v_s[128];
    __shared__ __align__(16) float red_r[8][128];
    __shared__ __align__(16) float red_o[8][128];
    __shared__ float ssum[4][2];
    __shared__ float osum[4];
    __shared__ float scal_s[2];

    const int tid = threadIdx.x, warp = tid >> 5, ln = tid & 31;
    const bool is_qv = tid < 128, issuer = warp == 4;
    const int c = tid & 127;
    // the grid is a multiple of 16, so a CTA keeps one head and strides over lanes
    const int h = blockIdx.x % kGdnHeads;
    const int lane_stride = gridDim.x / kGdnHeads;
    const uint32_t bar = smem_u32(&bar_storage);
    const uint32_t tile_addr = smem_u32(tile), in_addr = smem_u32(in_s);
    float nb_raw = 0.f, na_raw = 0.f;          // warp 4, lane 0: gate inputs of the item being fetched
    {
        const int l0 = blockIdx.x / kGdnHeads;
        if (tid == 0) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;\n" ::"r"(bar) : "memory");
            asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        }
        __syncthreads();
        // the first state tile is on its way before the projection kernel ahead of this one has ended
        if (tid == 128 && l0 < p.lanes) item_fetch(p, &pmap, &wmap0, &wmap1, &wmap2, l0, h, 1, tile_addr, in_addr, bar);
        pdl_wait();
        if (issuer && l0 < p.lanes) {
            if (ln == 0) {
                item_fetch(p, &pmap, &wmap0, &wmap1, &wmap2, l0, h, 2, tile_addr, in_addr, bar);
                const uint16_t* pr0 = p.proj + (size_t)l0 * p.T * kGdnProjN;
                nb_raw = bf2f(pr0[kOffB + h]);
                na_raw = bf2f(pr0[kOffA + h]);
            }
        }
    }

    // per-CTA constants of head h
    const float negA = -expf(bf2f(p.A_log[h]));
    const float dtb = bf2f(p.dt_bias[h]);
    const float q_scale = 0.08838834764831845f;   // 128^-1/2
    const int chA = (is_qv ? 0 : 2048) + h * 128 + c;          // q or k channel of this thread
    const int chB = 4096 + h * 128 + c;                        // v channel (warps 0-3)
    const uint2 tapA = *reinterpret_cast<const uint2*>(p.conv_w + (size_t)chA * 4);
    const uint2 tapB = *reinterpret_cast<const uint2*>(p.conv_w + (size_t)chB * 4);
    const float nw = bf2f(p.norm_w[c]);

    // gated RMSNorm of column c over the head's 128 outputs (f32 until the single bf16 cast); warps 4-7
    auto gated_norm = [&](float z, size_t row) {
        float o = 0.f;
#pragma unroll
        for (int w = 0; w < 8; ++w) o += red_o[w][c];
        const float oo = warp_sum(o * o);
        if (ln == 0) osum[warp - 4] = oo;
        asm volatile("bar.sync 3, 128;\n" ::: "memory");
        const float ms = (osum[0] + osum[1] + osum[2] + osum[3]) * (1.0f / 128.0f);
        float n = __fmul_rn(o, rsqrt_acc(ms + kEps));
        n = __fmul_rn(nw, n);
        p.y[row * kValueDim + h * 128 + c] = f2bf(__fmul_rn(n, silu_acc(z)));
    };

    uint32_t phase = 0;
    bool pend = false;                         // warps 4-7: a gated norm is owed for (row_pend, z_pend)
    size_t row_pend = 0;
    float z_pend = 0.f;
    for (int lane_id = blockIdx.x / kGdnHeads; lane_id < p.lanes; lane_id += lane_stride) {
        const int sel = p.sel != nullptr ? p.sel[lane_id] : 0;
        const size_t s_off = ((size_t)lane_id * kGdnHeads + h) * (kDk * kDv);
        const size_t w_off = (size_t)lane_id * 3 * kConvCh;
        float* S_live = pick_buf(p.S, sel) + s_off;
        uint16_t* win_live = pick_buf(p.win, sel) + w_off;

        // ---- prefetched tile and inputs: shared memory -> registers ------------------------------
        // one verdict for the whole CTA: nobody may leave while others go on to the barriers below
        if (!__syncthreads_and(mbar_wait_bounded(bar, phase))) {
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
        const int kindA = is_qv ? 0 : 1;
        float rawA = bf2f(in_s[kindA * 128 + c]), rawB = bf2f(in_s[2 * 128 + c]);
        float winA[3], winB[3];
#pragma unroll
        for (int j = 0; j < 3; ++j) {
            winA[j] = bf2f(in_s[(4 + j * 3 + kindA) * 128 + c]);
            winB[j] = bf2f(in_s[(4 + j * 3 + 2) * 128 + c]);
        }
        const float z_cur = bf2f(in_s[3 * 128 + c]);
        if (tid == 128) { scal_s[0] = nb_raw; scal_s[1] = na_raw; }
        // Every thread has its copy: the buffers are free again.  Only warp 4, which issues the next
        // fetch, waits for that; the others announce it and go on.
        if (issuer) {
            asm volatile("bar.sync 2, 256;\n" ::: "memory");
            const int nxt = lane_id + lane_stride;
            if (nxt < p.lanes) {
                if (ln == 0) {
                    item_fetch(p, &pmap, &wmap0, &wmap1, &wmap2, nxt, h, 3, tile_addr, in_addr, bar);
                    const uint16_t* prn = p.proj + (size_t)nxt * p.T * kGdnProjN;
                    nb_raw = bf2f(prn[kOffB + h]);
                    na_raw = bf2f(prn[kOffA + h]);
                }
            } else if (ln == 0) {
                pdl_trigger();             // last item of this CTA: the next kernel may start its weight loads
            }
        } else {
            asm volatile("bar.arrive 2, 256;\n" ::: "memory");
        }
        // the previous item's gated norm, in the shadow of this item's conv
        if (!is_qv && pend) {
            gated_norm(z_pend, row_pend);
            pend = false;
        }

        for (int t = 0; t < p.T; ++t) {
            const size_t row = (size_t)lane_id * p.T + t;
            const uint16_t* pr = p.proj + row * kGdnProjN;

            // ---- conv + SiLU: q and v on warps 0-3, k on warps 4-7 -------------------------------
            {
                if (t > 0) { rawA = bf2f(pr[chA]); rawB = bf2f(pr[chB]); }
                const float uA = conv_silu(winA, rawA, tapA);
                const float sq = warp_sum(uA * uA);
                if (is_qv) {
                    q_s[c] = uA;
                    v_s[c] = conv_silu(winB, rawB, tapB);
                    if (ln == 0) ssum[warp][0] = sq;
                } else {
                    k_s[c] = uA;
                    if (ln == 0) ssum[warp - 4][1] = sq;
                }
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

            // ---- gated RMSNorm: at once for a token that is not the item's last, else deferred ---
            if (!is_qv) {
                if (t + 1 < p.T) {
                    gated_norm(bf2f(pr[kOffZ + h * 128 + c]), row);
                } else {
                    pend = true;
                    row_pend = row;
                    z_pend = (t == 0) ? z_cur : bf2f(pr[kOffZ + h * 128 + c]);
                }
            }

            // ---- checkpoint after every non-final token of a speculative verify body -------------
            if (t < p.checkpoint) {
                int cb = sel + 1 + t;
                if (cb > p.checkpoint) cb -= p.checkpoint + 1;
                float4* Sc = reinterpret_cast<float4*>(pick_buf(p.S, cb) + s_off);
#pragma unroll
                for (int r = 0; r < 16; ++r) Sc[(warp * 16 + r) * 32 + ln] = s[r];
                uint16_t* wc = pick_buf(p.win, cb) + w_off;
#pragma unroll
                for (int j = 0; j < 3; ++j) {
                    wc[j * kConvCh + chA] = f2bf(winA[j]);
                    if (is_qv) wc[j * kConvCh + chB] = f2bf(winB[j]);
                }
            }
        }

        {
            float4* So = reinterpret_cast<float4*>(S_live);
#pragma unroll
            for (int r = 0; r < 16; ++r) So[(warp * 16 + r) * 32 + ln] = s[r];
        }
#pragma unroll
        for (int j = 0; j < 3; ++j) {
            win_live[j * kConvCh + chA] = f2bf(winA[j]);
            if (is_qv) win_live[j * kConvCh + chB] = f2bf(winB[j]);
        }
    }
    if (!is_qv && pend) gated_norm(z_pend, row_pend);      // the last item's norm
}

namespace {

// Tensor maps are pure functions of (base pointer, row count); a step uses the same few every time.
struct MapKey {
    const void* base;
    long long rows;
    int kind;
    bool operator==(const MapKey& o) const { return base == o.base && rows == o.rows && kind == o.kind; }
};
struct MapKeyHash {
    size_t operator()(const MapKey& k) const {
        return std::hash<const void*>()(k.base) ^ (std::hash<long long>()(k.rows) * 1315423911u) ^ (size_t)k.kind;
    }
};

// kind 0: projection rows [rows][8224] bf16 seen as {2048 inner, 4 pieces 2048 apart, rows}: box = the
//         128 values of one head in each of q, k, v, z.
// kind 1: conv windows [lanes][3 rows][6144] bf16 seen as {2048 inner, 3 kinds, 3 rows, lanes}: box = the
//         128 values of one head in each of the 3 x 3 (row, kind) pieces.
bool small_input_map(CUtensorMap* out, const uint16_t* base, long long rows, int kind) {
    static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
    static std::mutex mu;                       // engines of several host threads share this cache
    std::lock_guard<std::mutex> lock(mu);
    const MapKey key{base, rows, kind};
    auto it = cache.find(key);
    if (it != cache.end()) { *out = it->second; return true; }
    EncodeTiledFn fn = encode_tiled_fn();
    if (fn == nullptr || base == nullptr || rows <= 0) return false;
    CUresult r;
    if (kind == 0) {
        cuuint64_t dims[3] = {2048, 4, (cuuint64_t)rows};
        cuuint64_t strides[2] = {2048 * 2, (cuuint64_t)kGdnProjN * 2};
        cuuint32_t box[3] = {128, 4, 1}, elem[3] = {1, 1, 1};
        r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<uint16_t*>(base), dims, strides, box, elem,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    } else {
        cuuint64_t dims[4] = {2048, 3, 3, (cuuint64_t)rows};
        cuuint64_t strides[3] = {2048 * 2, (cuuint64_t)kConvCh * 2, (cuuint64_t)3 * kConvCh * 2};
        cuuint32_t box[4] = {128, 3, 3, 1}, elem[4] = {1, 1, 1, 1};
        r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<uint16_t*>(base), dims, strides, box, elem,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    }
    if (r != CUDA_SUCCESS) return false;
    if (cache.size() > 4096) cache.clear();
    cache.emplace(key, *out);
    return true;
}

}  // namespace

cudaError_t launch_gdn_step(const GdnParams& p, cudaStream_t st) {
    if (p.lanes <= 0 || p.T <= 0 || p.lanes > 65535) return cudaErrorInvalidValue;
    if (p.checkpoint < 0 || p.checkpoint >= kStateBufs) return cudaErrorInvalidValue;
    if (p.checkpoint > 0) {
        if (p.T != p.checkpoint + 1) return cudaErrorInvalidValue;
        for (int b = 0; b <= p.checkpoint; ++b)
            if (p.S[b] == nullptr || p.win[b] == nullptr) return cudaErrorInvalidValue;
    }
    static bool attr_done[kMaxDevices] = {false};           // per device
    {
        cudaError_t e = opt_in_smem(gdn_step_kernel, kGdnSmemBytes, attr_done);
        if (e != cudaSuccess) return e;
    }
    static int per_sm = 0;                                  // tuning knob, read once: Q35_GDN_CTAS_PER_SM = 1 or 2
    if (per_sm == 0) {
        const char* env = std::getenv("Q35_GDN_CTAS_PER_SM");
        per_sm = (env != nullptr && env[0] == '1') ? 1 : 2;
    }
    int max_ctas = (per_sm * sm_count() / kGdnHeads) * kGdnHeads;   // two CTAs per SM, rounded down to whole lanes
    if (max_ctas < kGdnHeads) max_ctas = kGdnHeads;
    const int items = p.lanes * kGdnHeads;
    const int grid = items < max_ctas ? items : max_ctas;
    CUtensorMap pmap, wmap[kStateBufs];
    if (!small_input_map(&pmap, p.proj, (long long)p.lanes * p.T, 0)) return cudaErrorInvalidValue;
    if (!small_input_map(&wmap[0], p.win[0], p.lanes, 1)) return cudaErrorInvalidValue;
    for (int b = 1; b < kStateBufs; ++b) {
        if (p.win[b] == nullptr) wmap[b] = wmap[0];
        else if (!small_input_map(&wmap[b], p.win[b], p.lanes, 1)) return cudaErrorInvalidValue;
    }
    return launch_k(gdn_step_kernel, dim3(grid), dim3(256), kGdnSmemBytes, st, p, pmap, wmap[0], wmap[1], wmap[2]);
}

}  // namespace q35
