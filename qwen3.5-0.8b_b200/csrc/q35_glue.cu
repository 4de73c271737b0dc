// Block glue: embedding gather, residual add + zero-centred RMSNorm, and the state-tuple
// layout converters.  Replaces glue_add_norm_rows / embed_gather_rows of the reference
// (engine/kernels.h:45, engine/kernels_embed.cpp:53-59).
#include "q35_common.cuh"

#include <cstdlib>

namespace q35 {

// Programmatic dependent launch pays where a body is a chain of short kernels (measured: 3-5 % of a
// step at 1-128 rows, a 2 % loss at 512).  Q35_PDL=1 / 0 forces it on / off; unset, a body of at
// most kPdlAutoRows rows turns it on for its own launches.
namespace {
constexpr int kPdlAutoRows = 192;
thread_local int g_pdl_rows = 1 << 30;      // per host thread: two engines driven by two threads do not share it
}
void pdl_set_rows(int rows) { g_pdl_rows = rows; }

int sm_count() {
    static int sms[kMaxDevices] = {0};
    const int dev = current_device_slot();
    if (dev < 0) return 148;
    if (sms[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        sms[dev] = n;
    }
    return sms[dev];
}
bool pdl_enabled() {
    static int v = -2;
    if (v == -2) {
        const char* e = std::getenv("Q35_PDL");
        v = (e == nullptr || e[0] == '\0') ? -1 : (e[0] == '1' ? 1 : 0);
    }
    return v >= 0 ? v == 1 : g_pdl_rows <= kPdlAutoRows;
}

// One warp per row of 1024: 32 lanes x 4 chunks of 8 bf16.  sum = bf16(x + delta) (bf16 add,
// one rounding), n = bf16( (sum * rsqrt(mean(sum^2) + eps)) * (1 + w) ) with f32 math in the
// reference's operation order (speccheck/specimpl.py:135-139).
__global__ void __launch_bounds__(256)
add_norm_kernel(const uint16_t* __restrict__ x, const int* __restrict__ ids,
                const uint16_t* __restrict__ table, int vocab, const uint16_t* __restrict__ delta,
                const uint16_t* __restrict__ w, uint16_t* __restrict__ sum_out,
                uint16_t* __restrict__ normed_out, int rows, const float* __restrict__ delta_parts,
                int n_split) {
    const int row = blockIdx.x * 8 + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    // the norm weights do not depend on the predecessor: fetch them ahead of the wait, off the chain
    uint4 wv[4];
#pragma unroll
    for (int c = 0; c < 4; ++c) wv[c] = *reinterpret_cast<const uint4*>(w + c * 256 + lane * 8);
    pdl_wait();
    pdl_trigger();          // the projection behind this kernel may start fetching its weights
    if (row >= rows) return;
    const uint16_t* src;
    if (ids != nullptr) {
        int id = ids[row];
        id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);   // ids are validated on the host; never read out of range
        src = table + (size_t)id * kHidden;
    } else {
        src = x + (size_t)row * kHidden;
    }
    float v[32];
    float ss = 0.f;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
        const int off = c * 256 + lane * 8;
        const uint4 a = *reinterpret_cast<const uint4*>(src + off);
        const uint32_t aw[4] = {a.x, a.y, a.z, a.w};
        uint32_t dw[4] = {0, 0, 0, 0};
        const bool has_delta = delta != nullptr || delta_parts != nullptr;
        if (delta != nullptr) {
            const uint4 d = *reinterpret_cast<const uint4*>(delta + (size_t)row * kHidden + off);
            dw[0] = d.x; dw[1] = d.y; dw[2] = d.z; dw[3] = d.w;
        } else if (delta_parts != nullptr) {
            // K-split projection: sum the partial tiles in split order, round once to bf16
            float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            for (int z = 0; z < n_split; ++z) {
                const float4* pp = reinterpret_cast<const float4*>(
                    delta_parts + ((size_t)z * rows + row) * kHidden + off);
                const float4 p0 = pp[0], p1 = pp[1];
                acc[0] += p0.x; acc[1] += p0.y; acc[2] += p0.z; acc[3] += p0.w;
                acc[4] += p1.x; acc[5] += p1.y; acc[6] += p1.z; acc[7] += p1.w;
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) dw[j] = pack_bf2(acc[2 * j], acc[2 * j + 1]);
        }
        uint32_t sw[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            float lo = lo_bf(aw[j]), hi = hi_bf(aw[j]);
            if (has_delta) {
                lo = bfround(lo + lo_bf(dw[j]));
                hi = bfround(hi + hi_bf(dw[j]));
            }
            v[c * 8 + 2 * j] = lo;
            v[c * 8 + 2 * j + 1] = hi;
            ss += lo * lo + hi * hi;
            sw[j] = pack_bf2(lo, hi);
        }
        if (sum_out != nullptr)
            *reinterpret_cast<uint4*>(sum_out + (size_t)row * kHidden + off) =
                make_uint4(sw[0], sw[1], sw[2], sw[3]);
    }
    ss = warp_sum(ss);
    const float inv = rsqrt_acc(ss * (1.0f / kHidden) + kEps);
    if (normed_out == nullptr) return;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
        const int off = c * 256 + lane * 8;
        const uint32_t ww[4] = {wv[c].x, wv[c].y, wv[c].z, wv[c].w};
        uint32_t o[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float lo = __fmul_rn(__fmul_rn(v[c * 8 + 2 * j], inv), 1.0f + lo_bf(ww[j]));
            const float hi = __fmul_rn(__fmul_rn(v[c * 8 + 2 * j + 1], inv), 1.0f + hi_bf(ww[j]));
            o[j] = pack_bf2(lo, hi);
        }
        *reinterpret_cast<uint4*>(normed_out + (size_t)row * kHidden + off) =
            make_uint4(o[0], o[1], o[2], o[3]);
    }
}

// K-split form: one CTA of 128 threads per row, 8 elements per thread, so the n_split f32 partial
// rows (4 KiB each) are pulled by many CTAs at once; the partial loads of up to eight splits are in flight
// together (eight, then four, then one).  Same arithmetic as add_norm_kernel (partials summed in split order, one bf16 rounding).
__global__ void __launch_bounds__(128)
add_norm_split_kernel(const uint16_t* __restrict__ x, const float* __restrict__ parts, int n_split,
                      const uint16_t* __restrict__ w, uint16_t* __restrict__ sum_out,
                      uint16_t* __restrict__ normed_out, int rows) {
    __shared__ float red[4];
    const int row = blockIdx.x, tid = threadIdx.x;
    const int off = tid * 8;
    const uint4 wv = *reinterpret_cast<const uint4*>(w + off);      // ahead of the wait: weights are immutable
    pdl_wait();
    pdl_trigger();          // the projection behind this kernel may start fetching its weights
    const uint4 a = *reinterpret_cast<const uint4*>(x + (size_t)row * kHidden + off);
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    const float* pp = parts + (size_t)row * kHidden + off;
    const size_t zs = (size_t)rows * kHidden;
    int z = 0;
    for (; z + 8 <= n_split; z += 8) {       // eight splits in flight: one round trip for most split counts
        float4 p[8][2];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            p[u][0] = *reinterpret_cast<const float4*>(pp + (z + u) * zs);
            p[u][1] = *reinterpret_cast<const float4*>(pp + (z + u) * zs + 4);
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            acc[0] += p[u][0].x; acc[1] += p[u][0].y; acc[2] += p[u][0].z; acc[3] += p[u][0].w;
            acc[4] += p[u][1].x; acc[5] += p[u][1].y; acc[6] += p[u][1].z; acc[7] += p[u][1].w;
        }
    }
    for (; z + 4 <= n_split; z += 4) {
        float4 p[4][2];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            p[u][0] = *reinterpret_cast<const float4*>(pp + (z + u) * zs);
            p[u][1] = *reinterpret_cast<const float4*>(pp + (z + u) * zs + 4);
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            acc[0] += p[u][0].x; acc[1] += p[u][0].y; acc[2] += p[u][0].z; acc[3] += p[u][0].w;
            acc[4] += p[u][1].x; acc[5] += p[u][1].y; acc[6] += p[u][1].z; acc[7] += p[u][1].w;
        }
    }
    for (; z < n_split; ++z) {
        const float4 p0 = *reinterpret_cast<const float4*>(pp + z * zs);
        const float4 p1 = *reinterpret_cast<const float4*>(pp + z * zs + 4);
        acc[0] += p0.x; acc[1] += p0.y; acc[2] += p0.z; acc[3] += p0.w;
        acc[4] += p1.x; acc[5] += p1.y; acc[6] += p1.z; acc[7] += p1.w;
    }
    const uint32_t aw[4] = {a.x, a.y, a.z, a.w};
    float v[8], ss = 0.f;
    uint32_t sw[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const float lo = bfround(lo_bf(aw[j]) + bfround(acc[2 * j]));
        const float hi = bfround(hi_bf(aw[j]) + bfround(acc[2 * j + 1]));
        v[2 * j] = lo; v[2 * j + 1] = hi;
        ss += lo * lo + hi * hi;
        sw[j] = pack_bf2(lo, hi);
    }
    if (sum_out != nullptr)
        *reinterpret_cast<uint4*>(sum_out + (size_t)row * kHidden + off) = make_uint4(sw[0], sw[1], sw[2], sw[3]);
    ss = warp_sum(ss);
    if ((tid & 31) == 0) red[tid >> 5] = ss;
    __syncthreads();
    const float inv = rsqrt_acc((red[0] + red[1] + red[2] + red[3]) * (1.0f / kHidden) + kEps);
    const uint32_t ww[4] = {wv.x, wv.y, wv.z, wv.w};
    uint32_t o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j)
        o[j] = pack_bf2(__fmul_rn(__fmul_rn(v[2 * j], inv), 1.0f + lo_bf(ww[j])),
                        __fmul_rn(__fmul_rn(v[2 * j + 1], inv), 1.0f + hi_bf(ww[j])));
    *reinterpret_cast<uint4*>(normed_out + (size_t)row * kHidden + off) = make_uint4(o[0], o[1], o[2], o[3]);
}

cudaError_t launch_add_norm(const uint16_t* x, const int* ids, const uint16_t* table, int vocab,
                            const uint16_t* delta, const uint16_t* w, uint16_t* sum_out,
                            uint16_t* normed_out, int rows, cudaStream_t st, const float* delta_parts,
                            int n_split) {
    if (w == nullptr) return cudaErrorInvalidValue;       // the kernels read the norm weights unconditionally
    if (delta_parts != nullptr && ids == nullptr && normed_out != nullptr)
        return launch_k(add_norm_split_kernel, dim3(rows), dim3(128), 0, st, x, delta_parts, n_split, w, sum_out,
                        normed_out, rows);
    return launch_k(add_norm_kernel, dim3((rows + 7) / 8), dim3(256), 0, st, x, ids, table, vocab, delta, w,
                    sum_out, normed_out, rows, delta_parts, n_split);
}

// ---- conv window: stored bf16 [3][6144] per (layer, lane); the reference layout is f32 ---------
__global__ void window_export_kernel(const uint16_t* __restrict__ win, float* __restrict__ out, int n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = bf2f(win[i]);
}
__global__ void window_import_kernel(const float* __restrict__ in, uint16_t* __restrict__ win, int n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) win[i] = f2bf(in[i]);
}
cudaError_t launch_window_export(const uint16_t* win, float* out, cudaStream_t st) {
    const int n = 3 * kConvCh;
    window_export_kernel<<<(n + 255) / 256, 256, 0, st>>>(win, out, n);
    return cudaGetLastError();
}
cudaError_t launch_window_import(const float* in, uint16_t* win, cudaStream_t st) {
    const int n = 3 * kConvCh;
    window_import_kernel<<<(n + 255) / 256, 256, 0, st>>>(in, win, n);
    return cudaGetLastError();
}

// ---- KV pages <-> contiguous [2][cap][256] (one layer, one lane, K or V) ------------------------
// grid (n_pos, 2 heads), 32 threads x 16 bytes = one 256-wide row
__global__ void kv_export_kernel(const uint16_t* __restrict__ pool, const int* __restrict__ table,
                                 int pages, uint16_t* __restrict__ out, int cap) {
    const int p = blockIdx.x, h = blockIdx.y;
    const int pg = p / kKvPage;
    if (pg >= pages || p >= cap) return;
    const uint16_t* src = pool + (size_t)table[pg] * kPageElems + ((size_t)h * kKvPage + p % kKvPage) * kHeadDim;
    uint16_t* dst = out + ((size_t)h * cap + p) * kHeadDim;
    reinterpret_cast<uint4*>(dst)[threadIdx.x] = reinterpret_cast<const uint4*>(src)[threadIdx.x];
}
__global__ void kv_import_kernel(const uint16_t* __restrict__ in, int cap, uint16_t* __restrict__ pool,
                                 const int* __restrict__ table, int pages) {
    const int p = blockIdx.x, h = blockIdx.y;
    const int pg = p / kKvPage;
    if (pg >= pages || p >= cap) return;
    uint16_t* dst = pool + (size_t)table[pg] * kPageElems + ((size_t)h * kKvPage + p % kKvPage) * kHeadDim;
    const uint16_t* src = in + ((size_t)h * cap + p) * kHeadDim;
    reinterpret_cast<uint4*>(dst)[threadIdx.x] = reinterpret_cast<const uint4*>(src)[threadIdx.x];
}
cudaError_t launch_kv_export(const uint16_t* pool, const int* table, int pages, uint16_t* out,
                             int cap, int n_pos, cudaStream_t st) {
    if (n_pos <= 0) return cudaSuccess;
    kv_export_kernel<<<dim3(n_pos, kKvHeads), 32, 0, st>>>(pool, table, pages, out, cap);
    return cudaGetLastError();
}
cudaError_t launch_kv_import(const uint16_t* in, int cap, int n_pos, uint16_t* pool, const int* table,
                             int pages, cudaStream_t st) {
    if (n_pos <= 0) return cudaSuccess;
    kv_import_kernel<<<dim3(n_pos, kKvHeads), 32, 0, st>>>(in, cap, pool, table, pages);
    return cudaGetLastError();
}

__global__ void fill_int_kernel(int* p, int v, int n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) p[i] = v;
}
__global__ void add_int_kernel(int* p, int v, int n) {
    pdl_wait();
    pdl_trigger();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) p[i] += v;
}
cudaError_t launch_fill_int(int* p, int v, int n, cudaStream_t st) {
    fill_int_kernel<<<(n + 255) / 256, 256, 0, st>>>(p, v, n);
    return cudaGetLastError();
}
cudaError_t launch_add_int(int* p, int v, int n, cudaStream_t st) {
    return launch_k(add_int_kernel, dim3((n + 255) / 256), dim3(256), 0, st, p, v, n);
}

}  // namespace q35
