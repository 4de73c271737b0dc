// Shared device helpers and launcher declarations for the sm_100a decode-path kernels.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace q35 {

constexpr int kLayers = 24;
constexpr int kGdnLayers = 18;
constexpr int kAttnLayers = 6;
constexpr int kHidden = 1024;
constexpr int kFF = 3584;
constexpr int kGdnHeads = 16;
constexpr int kDk = 128;
constexpr int kDv = 128;
constexpr int kConvCh = 6144;
constexpr int kValueDim = 2048;
constexpr int kGdnProjN = 8224;     // [qkv 6144 | z 2048 | b 16 | a 16]
constexpr int kQHeads = 8;
constexpr int kKvHeads = 2;
constexpr int kHeadDim = 256;
constexpr int kAttnProjN = 5120;    // [q|gate 4096 | k 512 | v 512]
constexpr int kRotHalf = 32;
constexpr int kKvPage = 64;
constexpr int kPageElems = kKvHeads * kKvPage * kHeadDim;   // bf16 elements per K (or V) page
constexpr float kEps = 1e-6f;

__host__ __device__ constexpr bool is_attn_layer(int l) { return l % 4 == 3; }

// ---- bf16 <-> f32 (round to nearest even; inputs are finite in this model) -------------------
__device__ __forceinline__ float bf2f(uint16_t b) { return __uint_as_float(((uint32_t)b) << 16); }
__device__ __forceinline__ uint16_t f2bf(float f) {
    return __bfloat16_as_ushort(__float2bfloat16_rn(f));
}
__device__ __forceinline__ float bfround(float f) { return bf2f(f2bf(f)); }
__device__ __forceinline__ float lo_bf(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float hi_bf(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }
__device__ __forceinline__ uint32_t pack_bf2(float lo, float hi) {
    return (uint32_t)f2bf(lo) | ((uint32_t)f2bf(hi) << 16);
}

// 1/sqrt(x) with IEEE sqrt and divide (the CPU reference's rsqrt is correctly rounded to ~1 ulp).
__device__ __forceinline__ float rsqrt_acc(float x) { return __fdiv_rn(1.0f, __fsqrt_rn(x)); }
__device__ __forceinline__ float sigmoid_acc(float x) { return __fdiv_rn(1.0f, 1.0f + expf(-x)); }
__device__ __forceinline__ float silu_acc(float x) { return __fdiv_rn(x, 1.0f + expf(-x)); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// ---- attention head helpers ----------------------------------------------------------------------
constexpr int kHeadDimC = 256;
__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
    f[0] = lo_bf(v.x); f[1] = hi_bf(v.x); f[2] = lo_bf(v.y); f[3] = hi_bf(v.y);
    f[4] = lo_bf(v.z); f[5] = hi_bf(v.z); f[6] = lo_bf(v.w); f[7] = hi_bf(v.w);
}

// Zero-centred RMSNorm of one 256-wide head held 8 values per lane, then partial RoPE.
// Returns the f32 result in x (rotated dims are NOT rounded; un-rotated dims are bf16 values).
// The norm weights and the lane's eight rotation frequencies are requested first, so their latency
// overlaps the reduction instead of following it.
__device__ __forceinline__ void head_norm_rope(float (&x)[8], const uint16_t* __restrict__ w, int ln,
                                               int rope_pos, const float* __restrict__ inv_freq) {
    const uint4 wv = *reinterpret_cast<const uint4*>(w + 8 * ln);
    // lanes 0..3 hold dims 0..31, lanes 4..7 hold dims 32..63; dim d rotates with frequency d & 31
    float4 f0 = make_float4(0.f, 0.f, 0.f, 0.f), f1 = f0;
    if (ln < 8) {
        const float4* fp = reinterpret_cast<const float4*>(inv_freq + ((8 * ln) & 31));
        f0 = fp[0];
        f1 = fp[1];
    }
    float ss = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) ss += x[e] * x[e];
    ss = warp_sum(ss);
    const float inv = rsqrt_acc(ss * (1.0f / kHeadDimC) + kEps);
    float wf[8];
    unpack8(wv, wf);
#pragma unroll
    for (int e = 0; e < 8; ++e) x[e] = bfround(__fmul_rn(__fmul_rn(x[e], inv), 1.0f + wf[e]));
    const float fr[8] = {f0.x, f0.y, f0.z, f0.w, f1.x, f1.y, f1.z, f1.w};
    // the partner of dim d is d ^ 32: four lanes away
#pragma unroll
    for (int e = 0; e < 8; ++e) {
        const float partner = __shfl_xor_sync(0xffffffffu, x[e], 4);
        if (ln < 8) {
            const float ang = __fmul_rn((float)rope_pos, fr[e]);
            float s, c;
            sincosf(ang, &s, &c);                 // one argument reduction for both
            const float sw = ln < 4 ? -partner : partner;
            x[e] = __fadd_rn(__fmul_rn(x[e], c), __fmul_rn(sw, s));
        }
    }
}

__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
    return make_uint4(pack_bf2(f[0], f[1]), pack_bf2(f[2], f[3]), pack_bf2(f[4], f[5]),
                      pack_bf2(f[6], f[7]));
}


// (value, index) with the greedy order: larger value wins, equal values -> lower index wins.
struct ArgMax {
    float v;
    int i;
};
__device__ __forceinline__ bool better(float av, int ai, float bv, int bi) {
    return av > bv || (av == bv && ai < bi);
}

// ---- programmatic dependent launch ---------------------------------------------------------------
// With Q35_PDL=1 every kernel of a body is launched with the programmatic-stream-serialization attribute: it may
// start while its predecessor drains.  A kernel calls pdl_wait() before it first touches anything an
// earlier kernel of the step wrote; before the wait it may only read what no kernel of the step
// writes (weights; the GDN state of the previous step).  pdl_trigger() comes LATE - once the kernel
// has issued its last loads, and always after its own wait - so at most one successor is resident
// beside its predecessor and everything older than the predecessor is complete.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;\n" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory"); }

// The TMA unit fetches a tensor map (128 bytes of kernel parameter space) on first use; asking for
// it at kernel entry takes that fetch off the first tile's critical path.
__device__ __forceinline__ void prefetch_tensormap(const void* map) {
    asm volatile("prefetch.tensormap [%0];\n" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

bool pdl_enabled();            // Q35_PDL=1/0 forces; unset: on for bodies of few rows (pdl_set_rows)
void pdl_set_rows(int rows);   // the engine announces the row count of the body it is about to launch (per host thread)

// ---- per-device facts ------------------------------------------------------------------------------
// Kernel attributes and the SM count belong to a device, not to the process: the flags and counts are
// kept per device ordinal (several engines on several devices may live in one process).
constexpr int kMaxDevices = 64;
int sm_count();                // multiprocessors of the current device
inline int current_device_slot() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return -1;
    return dev;
}
// opt a kernel in to `smem` bytes of dynamic shared memory, once per device
template <typename Kern>
inline cudaError_t opt_in_smem(Kern kern, size_t smem, bool (&done)[kMaxDevices]) {
    const int dev = current_device_slot();
    if (dev < 0) return cudaErrorInvalidDevice;
    if (!done[dev]) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
        done[dev] = true;
    }
    return cudaSuccess;
}

template <typename... KArgs, typename... Args>
inline cudaError_t launch_k(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                            Args&&... args) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}

// ---- launcher declarations (defined one per .cu file) -----------------------------------------
enum Epilogue { EPI_PLAIN = 0, EPI_SWIGLU = 1, EPI_ARGMAX = 2, EPI_PARTIAL = 3, EPI_RESID = 4 };

// out[rows][N] (or act / partial argmax) = x[rows][K] . W[N][K]^T, picks the few-row or tiled form.
// EPI_SWIGLU: W rows interleaved (2f gate, 2f+1 up), out [rows][N/2].
// EPI_ARGMAX: partials [rows][n_parts] ArgMax, logits (optional) f32 [rows][N]; returns n_parts.
cudaError_t launch_linear(const uint16_t* x, const uint16_t* W, void* out, int rows, int N, int K,
                          int epi, ArgMax* partials, float* logits, int* n_parts, cudaStream_t st,
                          int* status = nullptr);
const char* linear_route(int rows, int N, int K, int epi);      // name of the kernel launch_linear picks
const char* linear_tc_route(int rows, int N, int epi);
// tcgen05 / TMEM form (q35_gemm_tc.cu), taken by launch_linear for bodies of >= 64 rows
bool linear_tc_eligible(int rows, int N, int K);
// split-K route for narrow outputs at few rows: `splits` f32 partials [split][rows][N] in ws, which
// launch_add_norm sums (delta_parts).  linear_tc_splits returns 1 when the route does not apply.
constexpr int kMaxSplits = 16;
constexpr int kSplitMaxRows = 512;
int linear_tc_splits(int rows, int N, int K, int max_rows_ws);
cudaError_t launch_linear_tc_split(const uint16_t* x, const uint16_t* W, float* ws, int rows, int N, int K,
                                   int splits, int* status, cudaStream_t st);
cudaError_t launch_linear_tc(const uint16_t* x, const uint16_t* W, void* out, int rows, int N, int K, int epi,
                             ArgMax* partials, float* logits, int n_parts, int* status, cudaStream_t st);
int linear_argmax_parts(int rows, int N);
// Fused residual stream of bodies of at most kFusedMaxRows rows (the weight-streaming kernels): the
// output / down projection adds its result to the residual rows in place; the next in-projection /
// gate-up projection applies the RMSNorm (weights nw) while it stages those rows - every CTA holds all
// rows, so it takes their sums of squares from its own registers.  No add + norm kernel runs in between.
// pf / pf_bytes (optional): weights of a later kernel of the body, pulled into L2 by this one.
constexpr int kFusedMaxRows = 16;
cudaError_t launch_linear_resid_rows(const uint16_t* x, const uint16_t* W, uint16_t* resid, int rows, int K,
                                     const void* pf, size_t pf_bytes, cudaStream_t st);
cudaError_t launch_linear_norm_rows(const uint16_t* resid, const uint16_t* nw, const uint16_t* W, void* out, int rows,
                                    int N, int epi, const void* pf, size_t pf_bytes, cudaStream_t st);
cudaError_t launch_argmax_final(const ArgMax* partials, int n_parts, int rows, int* tokens,
                                float* top_logit, cudaStream_t st);
cudaError_t launch_pack_gate_up(const uint16_t* gate, const uint16_t* up, uint16_t* out,
                                cudaStream_t st);
// head + argmax for up to kStaticHeadMaxRows rows whose scratch is a fixed device array
constexpr int kStaticHeadMaxRows = 16;
constexpr int kStaticHeadMaxVocab = 262144;
cudaError_t launch_lm_head_static(const uint16_t* x, const uint16_t* embed, int vocab, int rows,
                                  int* tokens, cudaStream_t st);

// rows: sum = bf16(x + delta), normed = RMSNorm_zc(sum; w).  If ids != null, x row r is
// table[ids[r]] (embedding gather).  delta may be null.  row_map (optional) redirects reads:
// source row = row_map_stride * r + row_map_offset is expressed by the caller through pointers.
// delta_parts (optional, instead of delta): n_split f32 partials [n_split][rows][1024] whose sum,
// rounded once to bf16, is the delta.
cudaError_t launch_add_norm(const uint16_t* x, const int* ids, const uint16_t* table, int vocab,
                            const uint16_t* delta, const uint16_t* w, uint16_t* sum_out,
                            uint16_t* normed_out, int rows, cudaStream_t st,
                            const float* delta_parts = nullptr, int n_split = 0);

// Speculative verify keeps the state after each non-final row of its body in a shadow buffer, so a
// rejected candidate is undone by pointing the lane at another buffer: depth k needs k + 1 buffers.
constexpr int kStateBufs = 3;
template <typename T>
__host__ __device__ __forceinline__ T* pick_buf(T* const (&a)[kStateBufs], int i) {
    return i == 0 ? a[0] : (i == 1 ? a[1] : a[2]);      // selects, not an indexed copy of the parameter block
}

struct GdnParams {
    const uint16_t* proj;      // [lanes*T][8224]
    const uint16_t* conv_w;    // [6144][4]
    const uint16_t* A_log;     // [16]
    const uint16_t* dt_bias;   // [16]
    const uint16_t* norm_w;    // [128]
    float* S[kStateBufs];      // state buffers [lanes][16][128][128]; only S[0] must exist
    uint16_t* win[kStateBufs]; // window buffers [lanes][3][6144], allocated like S
    const int* sel;            // [lanes] live buffer index per lane, or null (= 0)
    uint16_t* y;               // [lanes*T][2048]
    int lanes, T;
    int checkpoint;            // c > 0: T == c + 1; the state after token t < c goes to buffer
                               // (sel + 1 + t) mod (c + 1), the state after the last token stays live
    int* status;               // device word raised to 1 if a bounded wait expires (may be null)
};
cudaError_t launch_gdn_step(const GdnParams& p, cudaStream_t st);
// chunk-64 form for bodies of many tokens per lane (no checkpoint); overwrites the raw q|k|v
// columns of p.proj with the conv outputs
constexpr int kGdnChunkMinT = 32;
cudaError_t launch_gdn_chunked(const GdnParams& p, cudaStream_t st);
cudaError_t gdn_chunk_init(cudaStream_t st);    // per-device lookup table of the chunked prefill; idempotent

struct AttnParams {
    const uint16_t* proj;      // [lanes*T][5120]
    const uint16_t* q_norm;    // [256]
    const uint16_t* k_norm;    // [256]
    uint16_t* kpool;           // pages [n_pages][2][64][256]
    uint16_t* vpool;
    const int* page_table;     // [lanes][pages_per_lane] page ids (for this layer)
    int pages_per_lane;
    long long table_lane_stride;  // ints between consecutive lanes in page_table
    const int* slot;           // [lanes] cache slot of the first new token (= positions cached)
    const int* rope_pos;       // [lanes] rope position of the first new token
    const float* inv_freq;     // [32]
    uint16_t* out;             // [lanes*T][2048]
    int lanes, T;
    int max_ctx;               // upper bound of slot + T over lanes (sizes shared memory)
    long long n_pages;         // pages in each pool (extent of the TMA tensor maps)
    const void* kmap;          // host CUtensorMap of kpool / vpool (attn_make_pool_map), or null:
    const void* vmap;          //   launch_attn then encodes them per call
    int* status;               // device word raised if a bounded wait expires (may be null)
};
constexpr int kTensorMapBytes = 128;
bool attn_make_pool_map(void* map_out, const uint16_t* pool, long long n_pages);
cudaError_t launch_attn(const AttnParams& p, cudaStream_t st);
cudaError_t attn_init();       // opt in to large dynamic shared memory; call once per device

// state tuple <-> reference layouts
cudaError_t launch_window_export(const uint16_t* win, float* out, cudaStream_t st);   // [3][6144]x18 handled by caller loop
cudaError_t launch_window_import(const float* in, uint16_t* win, cudaStream_t st);
cudaError_t launch_kv_export(const uint16_t* pool, const int* table, int pages, uint16_t* out,
                             int cap, int n_pos, cudaStream_t st);   // -> [2][cap][256]
cudaError_t launch_kv_import(const uint16_t* in, int cap, int n_pos, uint16_t* pool, const int* table,
                             int pages, cudaStream_t st);
cudaError_t launch_fill_int(int* p, int v, int n, cudaStream_t st);
cudaError_t launch_add_int(int* p, int v, int n, cudaStream_t st);

}  // namespace q35
