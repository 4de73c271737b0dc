// C-ABI of the decode engine: weight packing, scratch, the per-lane state tuple, and the
// decode / prefill / MTP bodies that chain the kernels of q35_{glue,gemm,gdn,attn}.cu.
// Interface contract: include/q35_engine.h.
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>

#include "../../include/q35_engine.h"
#include "q35_common.cuh"

using namespace q35;

// ------------------------------------------------------------------------------------------------
// errors
// ------------------------------------------------------------------------------------------------
static thread_local char g_err[512] = "";

static int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return code;
}
#define CK(call)                                                                                  \
    do {                                                                                          \
        cudaError_t _e = (call);                                                                  \
        if (_e != cudaSuccess)                                                                    \
            return fail(Q35_ERR_CUDA, "%s failed: %s (%s:%d)", #call, cudaGetErrorString(_e),     \
                        __FILE__, __LINE__);                                                      \
    } while (0)
#define REQUIRE(cond, code, ...)                                                                  \
    do {                                                                                          \
        if (!(cond)) return fail(code, __VA_ARGS__);                                              \
    } while (0)

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

extern "C" const char* q35_last_error(void) { return g_err; }
extern "C" int q35_abi_version(void) { return 1; }

// ------------------------------------------------------------------------------------------------
// objects
// ------------------------------------------------------------------------------------------------
struct PackedLayer {
    bool attn = false;
    uint16_t* in_w = nullptr;     // grouped in-projection [in_n][1024]
    int in_n = 0;
    uint16_t* out_w = nullptr;    // [1024][2048]
    uint16_t* gu_w = nullptr;     // interleaved gate/up [7168][1024]
    uint16_t* down_w = nullptr;   // [1024][3584]
    uint16_t* input_norm = nullptr;
    uint16_t* post_norm = nullptr;
    uint16_t *conv_w = nullptr, *A_log = nullptr, *dt_bias = nullptr, *gdn_norm = nullptr;
    uint16_t *q_norm = nullptr, *k_norm = nullptr;
};

struct q35_engine {
    q35_config cfg{};
    int vocab = 0, max_rows = 0;
    const uint16_t* embed = nullptr;
    uint16_t* final_norm = nullptr;
    PackedLayer layers[kLayers];
    bool has_mtp = false;
    uint16_t *mtp_fc = nullptr, *mtp_norm_emb = nullptr, *mtp_norm_hid = nullptr, *mtp_norm_out = nullptr;
    PackedLayer mtp_layer;
    // scratch, all [max_rows][...]
    uint16_t *resid = nullptr, *normed = nullptr, *proj = nullptr, *mix = nullptr, *delta = nullptr,
             *act = nullptr, *pair = nullptr, *last_normed = nullptr;
    ArgMax* partials = nullptr;
    int parts_cap = 0;
    int head_rows_cap = 0;                   // rows the head's partial-argmax scratch holds
    int *tok2 = nullptr, *tgt = nullptr;     // [max_rows] token scratch
    float* inv_freq = nullptr;
    int* dev_status = nullptr;               // raised by a kernel whose bounded wait expired
    float* split_ws = nullptr;               // [kMaxSplits][kSplitMaxRows][1024] f32 K-split partials
    bool l2_prefetch = true;                 // Q35_L2PF=0: few-row projections do not pull the next one's weights into L2
    bool fuse_enabled = true;                // Q35_FUSE=0: every body takes the add + norm kernels
    long long n_launch = 0;                  // kernels enqueued through this engine (captured ones count once)
    long long weight_bytes = 0;
    std::vector<void*> allocs;
    // optional per-family kernel timing (CUDA events on the launching stream)
    bool prof_on = false;
    std::vector<cudaEvent_t> prof_events;     // pairs: [2i] before, [2i+1] after
    std::vector<int> prof_family;
    size_t prof_used = 0;
    double prof_ms[Q35_FAMILIES] = {0};
    long long prof_launches[Q35_FAMILIES] = {0};
};

struct q35_state {
    q35_engine* e = nullptr;
    int lanes = 0, max_ctx = 0, pages_per_lane = 0;
    float* S[kStateBufs] = {nullptr, nullptr, nullptr};        // [18][lanes][16][128][128]; [1], [2]: MTP shadows
    uint16_t* win[kStateBufs] = {nullptr, nullptr, nullptr};   // [18][lanes][3][6144]
    int* sel = nullptr;                        // [lanes] live buffer per lane, allocated with the MTP shadow buffers
    uint16_t *kpool = nullptr, *vpool = nullptr;
    int* table = nullptr;                      // [lanes][6][pages_per_lane]
    int* pos = nullptr;                        // [lanes]
    int host_pos_hi = 0;                       // upper bound of any lane's position (host mirror)
    long long n_pages = 0;
    alignas(64) unsigned char kmap[kTensorMapBytes];   // TMA tensor maps of the two pools
    alignas(64) unsigned char vmap[kTensorMapBytes];
    std::vector<void*> allocs;
};

struct q35_mtp_state {
    q35_engine* e = nullptr;
    q35_state* s = nullptr;
    int lanes = 0, max_ctx = 0, pages_per_lane = 0;
    uint16_t *kpool = nullptr, *vpool = nullptr;
    int* table = nullptr;                      // [lanes][pages_per_lane]
    int* n = nullptr;                          // [lanes] rows in the draft cache
    int host_n_hi = 0;
    int drafts_pending = 0;                    // drafts enqueued since the last verify or reset (a verify of depth k needs k)
    int depth = 1;                             // candidates per round the shadow buffers allow
    uint16_t* h_tmp = nullptr;                 // [lanes][1024] a draft's output hidden, input of the next
    int* pos_tmp = nullptr;                    // [lanes]
    int* prop_tmp = nullptr;                   // [lanes]
    long long n_pages = 0;
    alignas(64) unsigned char kmap[kTensorMapBytes];
    alignas(64) unsigned char vmap[kTensorMapBytes];
    std::vector<void*> allocs;
};

template <typename T>
static cudaError_t dev_alloc(std::vector<void*>& owner, T** out, size_t count) {
    void* p = nullptr;
    cudaError_t e = cudaMalloc(&p, count * sizeof(T) > 0 ? count * sizeof(T) : 16);
    if (e != cudaSuccess) return e;
    owner.push_back(p);
    *out = static_cast<T*>(p);
    return cudaSuccess;
}
static void free_all(std::vector<void*>& owner) {
    for (void* p : owner) cudaFree(p);
    owner.clear();
}

// ------------------------------------------------------------------------------------------------
// small kernels that belong to the bodies
// ------------------------------------------------------------------------------------------------
// body ids of a verify round: row (lane, 0) = cur, rows (lane, 1..k) = the lane's candidates
__global__ void verify_ids_kernel(const int* __restrict__ cur, const int* __restrict__ cand, int k,
                                  int* __restrict__ out, int lanes) {
    pdl_wait();
    pdl_trigger();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= lanes * (k + 1)) return;
    const int lane_id = i / (k + 1), j = i % (k + 1);
    out[i] = j == 0 ? cur[lane_id] : cand[lane_id * k + j - 1];
}
__global__ void add_const_kernel(const int* __restrict__ in, int c, int* __restrict__ out, int n) {
    pdl_wait();
    pdl_trigger();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = in[i] + c;
}
__global__ void scatter_col_kernel(const int* __restrict__ in, int* __restrict__ out, int stride, int col, int n) {
    pdl_wait();
    pdl_trigger();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[(size_t)i * stride + col] = in[i];
}

// Accept rule of a depth-k round, all on the device (no host round trip): one warp per lane.
// tgt [lanes][k+1]: greedy ids of the body rows; cand [lanes][k].  The round accepts the LONGEST
// CORRECT PREFIX n of its candidates (engine/mtp_accept.h:113-123), emits cand[0..n) then tgt[n],
// and for n < k points the lane at the shadow buffer that holds the state after row n.  A round
// that did not accept everything also drops the k rows its drafts appended to the draft cache
// (speccheck/mtp.py:163-166).
__global__ void mtp_verdict_kernel(const int* __restrict__ cand, const int* __restrict__ tgt,
                                   const uint16_t* __restrict__ normed, int k, int* __restrict__ emit,
                                   int* __restrict__ n_emit, uint16_t* __restrict__ h_next,
                                   int* __restrict__ pos, int* __restrict__ sel,
                                   int* __restrict__ mtp_n, int lanes) {
    pdl_wait();
    pdl_trigger();          // the next round's first kernel may be set up; it reads what this one writes only after its own wait
    const int lane_id = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int ln = threadIdx.x & 31;
    if (lane_id >= lanes) return;
    const int* c = cand + (size_t)lane_id * k;
    const int* t = tgt + (size_t)lane_id * (k + 1);
    int n = 0;
    while (n < k && c[n] == t[n]) ++n;
    if (ln == 0) {
        int* em = emit + (size_t)lane_id * (k + 1);
        for (int i = 0; i <= k; ++i) em[i] = i < n ? c[i] : (i == n ? t[n] : -1);
        n_emit[lane_id] = n + 1;
        pos[lane_id] += n + 1;
        if (n < k) {
            int b = sel[lane_id] + 1 + n;
            if (b > k) b -= k + 1;
            sel[lane_id] = b;
            const int left = mtp_n[lane_id] - k;      // never below an empty cache, whatever order the host called in
            mtp_n[lane_id] = left > 0 ? left : 0;
        }
    }
    const uint4* src = reinterpret_cast<const uint4*>(normed + ((size_t)lane_id * (k + 1) + n) * kHidden);
    uint4* dst = reinterpret_cast<uint4*>(h_next + (size_t)lane_id * kHidden);
#pragma unroll
    for (int q = 0; q < 4; ++q) dst[q * 32 + ln] = src[q * 32 + ln];
}

// embedding gather for bodies whose ids are a [lanes][T_total] matrix and the body takes columns
// t0 .. t0+Tc-1: writes compact ids [lanes*Tc]
__global__ void slice_ids_kernel(const int* __restrict__ ids, int T_total, int t0, int Tc,
                                 int* __restrict__ out, int n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = ids[(size_t)(i / Tc) * T_total + t0 + (i % Tc)];
}

// ------------------------------------------------------------------------------------------------
// per-family kernel timing
// ------------------------------------------------------------------------------------------------
static cudaError_t prof_flush(q35_engine* e) {
    if (e->prof_used == 0) return cudaSuccess;
    cudaError_t ce = cudaEventSynchronize(e->prof_events[2 * e->prof_used - 1]);
    if (ce != cudaSuccess) return ce;
    for (size_t i = 0; i < e->prof_used; ++i) {
        float ms = 0.f;
        ce = cudaEventElapsedTime(&ms, e->prof_events[2 * i], e->prof_events[2 * i + 1]);
        if (ce != cudaSuccess) return ce;
        e->prof_ms[e->prof_family[i]] += ms;
        e->prof_launches[e->prof_family[i]] += 1;
    }
    e->prof_used = 0;
    return cudaSuccess;
}
static cudaError_t prof_begin(q35_engine* e, int family, cudaStream_t st) {
    if (e->prof_used >= 4096) {
        cudaError_t ce = prof_flush(e);
        if (ce != cudaSuccess) return ce;
    }
    while (e->prof_events.size() < 2 * (e->prof_used + 1)) {
        cudaEvent_t ev;
        cudaError_t ce = cudaEventCreate(&ev);
        if (ce != cudaSuccess) return ce;
        e->prof_events.push_back(ev);
    }
    if (e->prof_family.size() <= e->prof_used) e->prof_family.resize(e->prof_used + 1);
    e->prof_family[e->prof_used] = family;
    return cudaEventRecord(e->prof_events[2 * e->prof_used], st);
}
static cudaError_t prof_end(q35_engine* e, cudaStream_t st) {
    cudaError_t ce = cudaEventRecord(e->prof_events[2 * e->prof_used + 1], st);
    e->prof_used += 1;
    return ce;
}
// LAUNCH(family, call): CK(call), bracketed by events when timing is on
#define LAUNCH(family, call)                                  \
    do {                                                      \
        if (e->prof_on) CK(prof_begin(e, family, st));        \
        CK(call);                                             \
        e->n_launch += 1;                                     \
        if (e->prof_on) CK(prof_end(e, st));                  \
    } while (0)
// a kernel outside the families (token plumbing): counted, not timed
#define LAUNCH_PLAIN(call)                                    \
    do {                                                      \
        CK(call);                                             \
        e->n_launch += 1;                                     \
    } while (0)

extern "C" int q35_profile_begin(q35_engine* e) {
    REQUIRE(e, Q35_ERR_ARG, "q35_profile_begin: null engine");
    for (int f = 0; f < Q35_FAMILIES; ++f) { e->prof_ms[f] = 0; e->prof_launches[f] = 0; }
    e->prof_used = 0;
    e->prof_on = true;
    return Q35_OK;
}
extern "C" int q35_profile_end(q35_engine* e, double* ms_by_family, long long* launches_by_family) {
    REQUIRE(e && ms_by_family && launches_by_family, Q35_ERR_ARG, "q35_profile_end: null argument");
    e->prof_on = false;
    CK(prof_flush(e));
    for (int f = 0; f < Q35_FAMILIES; ++f) { ms_by_family[f] = e->prof_ms[f]; launches_by_family[f] = e->prof_launches[f]; }
    return Q35_OK;
}

// ------------------------------------------------------------------------------------------------
// engine
// ------------------------------------------------------------------------------------------------
static cudaError_t copy_rows(uint16_t* dst, const uint16_t* src, size_t elems, cudaStream_t st) {
    return cudaMemcpyAsync(dst, src, elems * sizeof(uint16_t), cudaMemcpyDeviceToDevice, st);
}

static int pack_layer(q35_engine* e, const q35_layer_weights& w, bool attn, PackedLayer* out,
                      cudaStream_t st, const char* what) {
    PackedLayer& L = *out;
    L.attn = attn;
    REQUIRE(w.input_norm && w.post_norm && w.mlp_gate && w.mlp_up && w.mlp_down, Q35_ERR_ARG,
            "%s: null norm / mlp weight", what);
    const size_t H = kHidden;
    if (attn) {
        REQUIRE(w.attn_q && w.attn_k && w.attn_v && w.attn_q_norm && w.attn_k_norm && w.attn_o,
                Q35_ERR_ARG, "%s: null attention weight", what);
        L.in_n = kAttnProjN;
        CK(dev_alloc(e->allocs, &L.in_w, (size_t)L.in_n * H));
        CK(copy_rows(L.in_w, w.attn_q, 4096 * H, st));
        CK(copy_rows(L.in_w + 4096 * H, w.attn_k, 512 * H, st));
        CK(copy_rows(L.in_w + 4608 * H, w.attn_v, 512 * H, st));
        CK(dev_alloc(e->allocs, &L.out_w, (size_t)kHidden * 2048));
        CK(copy_rows(L.out_w, w.attn_o, (size_t)kHidden * 2048, st));
        CK(dev_alloc(e->allocs, &L.q_norm, (size_t)kHeadDim));
        CK(dev_alloc(e->allocs, &L.k_norm, (size_t)kHeadDim));
        CK(copy_rows(L.q_norm, w.attn_q_norm, kHeadDim, st));
        CK(copy_rows(L.k_norm, w.attn_k_norm, kHeadDim, st));
    } else {
        REQUIRE(w.gdn_in_qkv && w.gdn_in_z && w.gdn_in_b && w.gdn_in_a && w.gdn_conv && w.gdn_A_log &&
                    w.gdn_dt_bias && w.gdn_norm && w.gdn_out,
                Q35_ERR_ARG, "%s: null GDN weight", what);
        L.in_n = kGdnProjN;
        CK(dev_alloc(e->allocs, &L.in_w, (size_t)L.in_n * H));
        CK(copy_rows(L.in_w, w.gdn_in_qkv, 6144 * H, st));
        CK(copy_rows(L.in_w + 6144 * H, w.gdn_in_z, 2048 * H, st));
        CK(copy_rows(L.in_w + 8192 * H, w.gdn_in_b, 16 * H, st));
        CK(copy_rows(L.in_w + 8208 * H, w.gdn_in_a, 16 * H, st));
        CK(dev_alloc(e->allocs, &L.out_w, (size_t)kHidden * 2048));
        CK(copy_rows(L.out_w, w.gdn_out, (size_t)kHidden * 2048, st));
        CK(dev_alloc(e->allocs, &L.conv_w, (size_t)kConvCh * 4));
        CK(copy_rows(L.conv_w, w.gdn_conv, (size_t)kConvCh * 4, st));
        CK(dev_alloc(e->allocs, &L.A_log, (size_t)16));
        CK(dev_alloc(e->allocs, &L.dt_bias, (size_t)16));
        CK(dev_alloc(e->allocs, &L.gdn_norm, (size_t)128));
        CK(copy_rows(L.A_log, w.gdn_A_log, 16, st));
        CK(copy_rows(L.dt_bias, w.gdn_dt_bias, 16, st));
        CK(copy_rows(L.gdn_norm, w.gdn_norm, 128, st));
    }
    CK(dev_alloc(e->allocs, &L.gu_w, (size_t)2 * kFF * H));
    CK(launch_pack_gate_up(w.mlp_gate, w.mlp_up, L.gu_w, st));
    CK(dev_alloc(e->allocs, &L.down_w, (size_t)kHidden * kFF));
    CK(copy_rows(L.down_w, w.mlp_down, (size_t)kHidden * kFF, st));
    CK(dev_alloc(e->allocs, &L.input_norm, H));
    CK(dev_alloc(e->allocs, &L.post_norm, H));
    CK(copy_rows(L.input_norm, w.input_norm, H, st));
    CK(copy_rows(L.post_norm, w.post_norm, H, st));
    e->weight_bytes += 2LL * ((long long)L.in_n * H + 2048LL * H + 2LL * kFF * H + (long long)kFF * H + 2 * H);
    e->weight_bytes += attn ? 2LL * 2 * kHeadDim : 2LL * (kConvCh * 4 + 16 + 16 + 128);
    return Q35_OK;
}

static int engine_build(q35_engine* e, const q35_config* cfg, const q35_weights* w, cudaStream_t st) {
    e->cfg = *cfg;
    {
        const char* env = getenv("Q35_FUSE");
        e->fuse_enabled = !(env != nullptr && env[0] == '0');
        env = getenv("Q35_L2PF");
        e->l2_prefetch = !(env != nullptr && env[0] == '0');
    }
    e->vocab = cfg->vocab;
    e->max_rows = cfg->max_rows;
    e->embed = w->embed;
    CK(attn_init());
    CK(gdn_chunk_init(st));
    CK(dev_alloc(e->allocs, &e->final_norm, (size_t)kHidden));
    CK(copy_rows(e->final_norm, w->final_norm, kHidden, st));
    e->weight_bytes = 2LL * e->vocab * kHidden + 2LL * kHidden;
    for (int l = 0; l < kLayers; ++l) {
        char what[32];
        snprintf(what, sizeof(what), "layer %d", l);
        int rc = pack_layer(e, w->layers[l], is_attn_layer(l), &e->layers[l], st, what);
        if (rc != Q35_OK) return rc;
    }
    e->has_mtp = w->has_mtp != 0;
    if (e->has_mtp) {
        REQUIRE(w->mtp.fc && w->mtp.norm_emb && w->mtp.norm_hid && w->mtp.norm_out, Q35_ERR_ARG,
                "mtp: null weight");
        const long long before = e->weight_bytes;
        int rc = pack_layer(e, w->mtp.layer, true, &e->mtp_layer, st, "mtp layer");
        if (rc != Q35_OK) return rc;
        e->weight_bytes = before;   // the census counts the target step only
        CK(dev_alloc(e->allocs, &e->mtp_fc, (size_t)kHidden * 2048));
        CK(copy_rows(e->mtp_fc, w->mtp.fc, (size_t)kHidden * 2048, st));
        CK(dev_alloc(e->allocs, &e->mtp_norm_emb, (size_t)kHidden));
        CK(dev_alloc(e->allocs, &e->mtp_norm_hid, (size_t)kHidden));
        CK(dev_alloc(e->allocs, &e->mtp_norm_out, (size_t)kHidden));
        CK(copy_rows(e->mtp_norm_emb, w->mtp.norm_emb, kHidden, st));
        CK(copy_rows(e->mtp_norm_hid, w->mtp.norm_hid, kHidden, st));
        CK(copy_rows(e->mtp_norm_out, w->mtp.norm_out, kHidden, st));
    }
    const size_t R = (size_t)e->max_rows;
    e->head_rows_cap = e->max_rows < 16384 ? e->max_rows : 16384;   // the head sees lanes (or 2 x lanes) rows, never a whole prefill body
    CK(dev_alloc(e->allocs, &e->resid, R * kHidden));
    CK(dev_alloc(e->allocs, &e->normed, R * kHidden));
    CK(dev_alloc(e->allocs, &e->proj, R * kGdnProjN));
    CK(dev_alloc(e->allocs, &e->mix, R * 2048));
    CK(dev_alloc(e->allocs, &e->delta, R * kHidden));
    CK(dev_alloc(e->allocs, &e->act, R * kFF));
    CK(dev_alloc(e->allocs, &e->pair, (e->has_mtp ? (size_t)e->head_rows_cap : 1) * 2048));
    CK(dev_alloc(e->allocs, &e->last_normed, R * kHidden));
    e->parts_cap = (e->vocab + 31) / 32;
    CK(dev_alloc(e->allocs, &e->partials, (size_t)e->head_rows_cap * e->parts_cap));
    CK(dev_alloc(e->allocs, &e->tok2, R));
    CK(dev_alloc(e->allocs, &e->tgt, R));
    CK(dev_alloc(e->allocs, &e->inv_freq, (size_t)32));
    CK(dev_alloc(e->allocs, &e->split_ws, (size_t)kMaxSplits * kSplitMaxRows * kHidden));
    CK(dev_alloc(e->allocs, &e->dev_status, (size_t)4));
    CK(cudaMemsetAsync(e->dev_status, 0, 4 * sizeof(int), st));
    CK(cudaMemcpyAsync(e->inv_freq, e->cfg.rope_inv_freq, 32 * sizeof(float), cudaMemcpyHostToDevice, st));
    CK(cudaStreamSynchronize(st));   // the host-side config copy above must not outlive `cfg`
    return Q35_OK;
}

extern "C" int q35_engine_create(const q35_config* cfg, const q35_weights* w, void* stream,
                                 q35_engine** out) {
    REQUIRE(cfg && w && out, Q35_ERR_ARG, "q35_engine_create: null argument");
    REQUIRE(cfg->vocab >= 8 && cfg->vocab % 8 == 0, Q35_ERR_ARG, "vocab %d must be a positive multiple of 8", cfg->vocab);
    REQUIRE(cfg->max_rows >= 1 && cfg->max_rows <= (1 << 20), Q35_ERR_ARG, "max_rows %d out of range", cfg->max_rows);
    REQUIRE(w->embed && w->final_norm && aligned16(w->embed), Q35_ERR_ARG, "embed / final_norm null or misaligned");
    q35_engine* e = new q35_engine();
    int rc = engine_build(e, cfg, w, static_cast<cudaStream_t>(stream));
    if (rc != Q35_OK) {
        free_all(e->allocs);
        delete e;
        return rc;
    }
    *out = e;
    return Q35_OK;
}

extern "C" int q35_engine_destroy(q35_engine* e) {
    if (!e) return Q35_OK;
    for (cudaEvent_t ev : e->prof_events) cudaEventDestroy(ev);
    free_all(e->allocs);
    delete e;
    return Q35_OK;
}

extern "C" int q35_engine_status(q35_engine* e, int* status_host) {
    REQUIRE(e && status_host, Q35_ERR_ARG, "q35_engine_status: null argument");
    CK(cudaMemcpy(status_host, e->dev_status, sizeof(int), cudaMemcpyDeviceToHost));
    return Q35_OK;
}

extern "C" int q35_step_census(const q35_engine* e, q35_census* out) {
    REQUIRE(e && out, Q35_ERR_ARG, "q35_step_census: null argument");
    out->weight_bytes = e->weight_bytes;
    out->lane_state_bytes = 2LL * kGdnLayers * kGdnHeads * kDk * kDv * 4 + 4LL * kGdnLayers * kConvCh * 4;
    out->kv_bytes_per_pos = 2LL * kAttnLayers * kKvHeads * kHeadDim * 2;
    long long params = 0;
    for (int l = 0; l < kLayers; ++l)
        params += ((long long)e->layers[l].in_n + 2048 + 3LL * kFF) * kHidden;
    params += (long long)e->vocab * kHidden;
    out->flops_per_row = 2 * params;
    out->launches_decode = 1 + kLayers * 7 + 3;                                  // bodies beyond the fused row limit
    out->launches_decode_few_lanes = e->fuse_enabled ? 1 + kLayers * 5 + 1 + 3 : out->launches_decode;
    return Q35_OK;
}

// ------------------------------------------------------------------------------------------------
// state
// ------------------------------------------------------------------------------------------------
extern "C" int q35_state_sizes_of(int lanes, int max_ctx, q35_state_sizes* out) {
    REQUIRE(out && lanes >= 1 && max_ctx >= 1, Q35_ERR_ARG, "q35_state_sizes_of: bad argument");
    const size_t pages = (size_t)(max_ctx + kKvPage - 1) / kKvPage;
    out->gdn_state_bytes = (size_t)kGdnLayers * kGdnHeads * kDk * kDv * sizeof(float);
    out->conv_window_bytes = (size_t)kGdnLayers * 3 * kConvCh * sizeof(uint16_t);
    out->kv_bytes = 2 * (size_t)kAttnLayers * pages * kPageElems * sizeof(uint16_t);
    out->per_token_bytes = 2 * (size_t)kAttnLayers * kKvHeads * kHeadDim * sizeof(uint16_t);
    out->total_bytes = (size_t)lanes * (out->gdn_state_bytes + out->conv_window_bytes + out->kv_bytes);
    return Q35_OK;
}

extern "C" int q35_state_reset(q35_state* s, void* stream) {
    REQUIRE(s, Q35_ERR_ARG, "q35_state_reset: null state");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const size_t sn = (size_t)kGdnLayers * s->lanes * kGdnHeads * kDk * kDv;
    const size_t wn = (size_t)kGdnLayers * s->lanes * 3 * kConvCh;
    for (int b = 0; b < kStateBufs; ++b) {
        if (s->S[b]) CK(cudaMemsetAsync(s->S[b], 0, sn * sizeof(float), st));
        if (s->win[b]) CK(cudaMemsetAsync(s->win[b], 0, wn * sizeof(uint16_t), st));
    }
    if (s->sel) CK(cudaMemsetAsync(s->sel, 0, s->lanes * sizeof(int), st));
    CK(cudaMemsetAsync(s->pos, 0, s->lanes * sizeof(int), st));
    s->host_pos_hi = 0;
    return Q35_OK;
}

extern "C" int q35_state_create(q35_engine* e, int lanes, int max_ctx, q35_state** out) {
    REQUIRE(e && out, Q35_ERR_ARG, "q35_state_create: null argument");
    REQUIRE(lanes >= 1 && lanes <= e->max_rows, Q35_ERR_CAPACITY, "lanes %d exceeds engine max_rows %d", lanes, e->max_rows);
    REQUIRE(max_ctx >= 1 && max_ctx <= 8192, Q35_ERR_CAPACITY, "max_ctx %d out of range [1, 8192]", max_ctx);
    q35_state* s = new q35_state();
    s->e = e;
    s->lanes = lanes;
    s->max_ctx = max_ctx;
    s->pages_per_lane = (max_ctx + kKvPage - 1) / kKvPage;
    const size_t sn = (size_t)kGdnLayers * lanes * kGdnHeads * kDk * kDv;
    const size_t wn = (size_t)kGdnLayers * lanes * 3 * kConvCh;
    const size_t n_pages = (size_t)lanes * kAttnLayers * s->pages_per_lane;
    cudaError_t ce = cudaSuccess;
    if (ce == cudaSuccess) ce = dev_alloc(s->allocs, &s->S[0], sn);
    if (ce == cudaSuccess) ce = dev_alloc(s->allocs, &s->win[0], wn);
    if (ce == cudaSuccess) ce = dev_alloc(s->allocs, &s->kpool, n_pages * kPageElems);
    if (ce == cudaSuccess) ce = dev_alloc(s->allocs, &s->vpool, n_pages * kPageElems);
    if (ce == cudaSuccess) ce = dev_alloc(s->allocs, &s->table, n_pages);
    if (ce == cudaSuccess) ce = dev_alloc(s->allocs, &s->pos, (size_t)lanes);
    s->n_pages = (long long)n_pages;
    if (ce == cudaSuccess && (!attn_make_pool_map(s->kmap, s->kpool, s->n_pages) ||
                              !attn_make_pool_map(s->vmap, s->vpool, s->n_pages)))
        ce = cudaErrorInvalidValue;
    if (ce == cudaSuccess) {
        // identity page map: lane-major, then layer, then page (any permutation is legal)
        std::vector<int> t(n_pages);
        for (size_t i = 0; i < n_pages; ++i) t[i] = (int)i;
        ce = cudaMemcpy(s->table, t.data(), n_pages * sizeof(int), cudaMemcpyHostToDevice);
    }
    if (ce == cudaSuccess) ce = cudaMemset(s->kpool, 0, n_pages * kPageElems * sizeof(uint16_t));
    if (ce == cudaSuccess) ce = cudaMemset(s->vpool, 0, n_pages * kPageElems * sizeof(uint16_t));
    int rc = Q35_OK;
    if (ce != cudaSuccess) rc = fail(Q35_ERR_CUDA, "q35_state_create: %s", cudaGetErrorString(ce));
    if (rc == Q35_OK) rc = q35_state_reset(s, nullptr);
    if (rc == Q35_OK && cudaDeviceSynchronize() != cudaSuccess) rc = fail(Q35_ERR_CUDA, "q35_state_create: sync failed");
    if (rc != Q35_OK) {
        free_all(s->allocs);
        delete s;
        return rc;
    }
    *out = s;
    return Q35_OK;
}

extern "C" int q35_state_destroy(q35_state* s) {
    if (!s) return Q35_OK;
    free_all(s->allocs);
    delete s;
    return Q35_OK;
}

extern "C" int q35_state_positions(q35_state* s, int* positions_out, void* stream) {
    REQUIRE(s && positions_out, Q35_ERR_ARG, "q35_state_positions: null argument");
    CK(cudaMemcpyAsync(positions_out, s->pos, s->lanes * sizeof(int), cudaMemcpyDeviceToDevice,
                       static_cast<cudaStream_t>(stream)));
    return Q35_OK;
}

// The host keeps an upper bound of the lanes' positions for capacity checks.  A caller that
// replays a captured CUDA graph of n steps reports them here (the captured call counted once).
extern "C" int q35_state_note_advance(q35_state* s, int n) {
    REQUIRE(s, Q35_ERR_ARG, "q35_state_note_advance: null state");
    REQUIRE(s->host_pos_hi + n <= s->max_ctx && s->host_pos_hi + n >= 0, Q35_ERR_CAPACITY,
            "position %d + %d beyond max_ctx %d", s->host_pos_hi, n, s->max_ctx);
    s->host_pos_hi += n;
    return Q35_OK;
}

// Speculative rounds advance a lane by 1..k+1 positions and the host cannot know by how many without
// reading back, so its bound moves by the maximum every round.  This call reads the true positions
// (one small copy and a stream synchronisation) and tightens the bound to their maximum.
extern "C" int q35_state_sync_bound(q35_state* s, void* stream) {
    REQUIRE(s, Q35_ERR_ARG, "q35_state_sync_bound: null state");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    std::vector<int> pos(s->lanes);
    CK(cudaMemcpyAsync(pos.data(), s->pos, s->lanes * sizeof(int), cudaMemcpyDeviceToHost, st));
    CK(cudaStreamSynchronize(st));
    int hi = 0;
    for (int v : pos) hi = v > hi ? v : hi;
    s->host_pos_hi = hi;
    return Q35_OK;
}

static int host_sel(q35_state* s, int lane, cudaStream_t st, int* out) {
    *out = 0;
    if (s->sel) {
        CK(cudaMemcpyAsync(out, s->sel + lane, sizeof(int), cudaMemcpyDeviceToHost, st));
        CK(cudaStreamSynchronize(st));
        if (*out < 0 || *out >= kStateBufs || s->S[*out] == nullptr) return fail(Q35_ERR_STATE, "lane %d selects a state buffer that does not exist", lane);
    }
    return Q35_OK;
}

extern "C" int q35_state_export_lane(q35_state* s, int lane, float* gdn_state, float* conv_window,
                                     uint16_t* kv_keys, uint16_t* kv_values, int cap, void* stream) {
    REQUIRE(s && lane >= 0 && lane < s->lanes, Q35_ERR_ARG, "q35_state_export_lane: bad lane");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    int b = 0;
    int rc = host_sel(s, lane, st, &b);
    if (rc != Q35_OK) return rc;
    const size_t per = (size_t)kGdnHeads * kDk * kDv;
    for (int g = 0; g < kGdnLayers; ++g) {
        if (gdn_state)
            CK(cudaMemcpyAsync(gdn_state + g * per, s->S[b] + ((size_t)g * s->lanes + lane) * per,
                               per * sizeof(float), cudaMemcpyDeviceToDevice, st));
        if (conv_window)
            CK(launch_window_export(s->win[b] + ((size_t)g * s->lanes + lane) * 3 * kConvCh,
                                    conv_window + (size_t)g * 3 * kConvCh, st));
    }
    if (kv_keys || kv_values) {
        REQUIRE(cap >= 1, Q35_ERR_ARG, "q35_state_export_lane: cap %d", cap);
        const int n_pos = cap < s->max_ctx ? cap : s->max_ctx;
        for (int a = 0; a < kAttnLayers; ++a) {
            const int* tb = s->table + ((size_t)lane * kAttnLayers + a) * s->pages_per_lane;
            if (kv_keys) CK(launch_kv_export(s->kpool, tb, s->pages_per_lane, kv_keys + (size_t)a * 2 * cap * kHeadDim, cap, n_pos, st));
            if (kv_values) CK(launch_kv_export(s->vpool, tb, s->pages_per_lane, kv_values + (size_t)a * 2 * cap * kHeadDim, cap, n_pos, st));
        }
    }
    return Q35_OK;
}

extern "C" int q35_state_import_lane(q35_state* s, int lane, const float* gdn_state,
                                     const float* conv_window, const uint16_t* kv_keys,
                                     const uint16_t* kv_values, int cap, int prefix_len, void* stream) {
    REQUIRE(s && lane >= 0 && lane < s->lanes, Q35_ERR_ARG, "q35_state_import_lane: bad lane");
    REQUIRE(prefix_len >= 0 && prefix_len <= s->max_ctx, Q35_ERR_CAPACITY, "prefix_len %d beyond max_ctx %d", prefix_len, s->max_ctx);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    int b = 0;
    int rc = host_sel(s, lane, st, &b);
    if (rc != Q35_OK) return rc;
    const size_t per = (size_t)kGdnHeads * kDk * kDv;
    for (int g = 0; g < kGdnLayers; ++g) {
        if (gdn_state)
            CK(cudaMemcpyAsync(s->S[b] + ((size_t)g * s->lanes + lane) * per, gdn_state + g * per,
                               per * sizeof(float), cudaMemcpyDeviceToDevice, st));
        if (conv_window)
            CK(launch_window_import(conv_window + (size_t)g * 3 * kConvCh,
                                    s->win[b] + ((size_t)g * s->lanes + lane) * 3 * kConvCh, st));
    }
    if (kv_keys || kv_values) {
        REQUIRE(cap >= prefix_len, Q35_ERR_ARG, "q35_state_import_lane: cap %d < prefix_len %d", cap, prefix_len);
        for (int a = 0; a < kAttnLayers; ++a) {
            const int* tb = s->table + ((size_t)lane * kAttnLayers + a) * s->pages_per_lane;
            if (kv_keys) CK(launch_kv_import(kv_keys + (size_t)a * 2 * cap * kHeadDim, cap, prefix_len, s->kpool, tb, s->pages_per_lane, st));
            if (kv_values) CK(launch_kv_import(kv_values + (size_t)a * 2 * cap * kHeadDim, cap, prefix_len, s->vpool, tb, s->pages_per_lane, st));
        }
    }
    CK(launch_fill_int(s->pos + lane, prefix_len, 1, st));
    if (prefix_len > s->host_pos_hi) s->host_pos_hi = prefix_len;
    return Q35_OK;
}

// ------------------------------------------------------------------------------------------------
// the body: `T` tokens per lane through the 24 blocks (T = 1 is the decode step)
// ------------------------------------------------------------------------------------------------
// Whether a body of `rows` rows takes the fused residual stream: the output / down projections add
// into the residual rows in place, the next projection applies the RMSNorm while it stages its rows,
// and the 48 add + norm kernels of a body do not run.
static bool body_fused(const q35_engine* e, int rows) { return e->fuse_enabled && rows <= kFusedMaxRows; }

// One block l over `rows` = lanes x T rows.  On entry the residual rows are in e->resid; the normed
// rows the in-projection reads are in e->normed when `in_from_normed`, else (fused stream) they are
// formed from e->resid while the projection stages them.  On exit e->resid holds the block's output
// rows; in the unfused form e->normed also holds them normed with `next_norm`.
static int run_layer(q35_engine* e, q35_state* s, int l, int T, int checkpoint, bool fused, bool in_from_normed,
                     const uint16_t* next_norm, const void* next_w, size_t next_w_bytes, cudaStream_t st) {
    const int rows = s->lanes * T;
    const PackedLayer& L = e->layers[l];
    // weights a projection pulls into L2 for the projection after it (few-row bodies only)
    const bool pf = e->l2_prefetch && fused;
    const size_t out_bytes = (size_t)kHidden * 2048 * 2, gu_bytes = (size_t)2 * kFF * kHidden * 2, down_bytes = (size_t)kHidden * kFF * 2;
    int gslot = 0, aslot = 0;
    for (int i = 0; i < l; ++i) (is_attn_layer(i) ? aslot : gslot) += 1;
    if (in_from_normed)
        LAUNCH(Q35_FAM_IN_PROJ, launch_linear(e->normed, L.in_w, e->proj, rows, L.in_n, kHidden, EPI_PLAIN, nullptr, nullptr, nullptr, st, e->dev_status));
    else
        LAUNCH(Q35_FAM_IN_PROJ, launch_linear_norm_rows(e->resid, L.input_norm, L.in_w, e->proj, rows, L.in_n, EPI_PLAIN,
                                                        pf ? L.out_w : nullptr, out_bytes, st));
    if (L.attn) {
        AttnParams ap{};
        ap.proj = e->proj; ap.q_norm = L.q_norm; ap.k_norm = L.k_norm;
        ap.kpool = s->kpool; ap.vpool = s->vpool;
        ap.page_table = s->table + (size_t)aslot * s->pages_per_lane;
        ap.pages_per_lane = s->pages_per_lane;
        ap.table_lane_stride = (long long)kAttnLayers * s->pages_per_lane;
        ap.slot = s->pos; ap.rope_pos = s->pos; ap.inv_freq = e->inv_freq;
        ap.out = e->mix; ap.lanes = s->lanes; ap.T = T; ap.max_ctx = s->max_ctx;
        ap.n_pages = s->n_pages; ap.kmap = s->kmap; ap.vmap = s->vmap; ap.status = e->dev_status;
        LAUNCH(Q35_FAM_ATTN, launch_attn(ap, st));
    } else {
        GdnParams gp{};
        gp.proj = e->proj; gp.conv_w = L.conv_w; gp.A_log = L.A_log; gp.dt_bias = L.dt_bias;
        gp.norm_w = L.gdn_norm;
        const size_t so = (size_t)gslot * s->lanes * kGdnHeads * kDk * kDv;
        const size_t wo = (size_t)gslot * s->lanes * 3 * kConvCh;
        for (int b = 0; b < kStateBufs; ++b) {
            gp.S[b] = s->S[b] ? s->S[b] + so : nullptr;
            gp.win[b] = s->win[b] ? s->win[b] + wo : nullptr;
        }
        gp.sel = s->sel; gp.y = e->mix; gp.lanes = s->lanes; gp.T = T; gp.checkpoint = checkpoint;
        gp.status = e->dev_status;
        if (!checkpoint && T >= kGdnChunkMinT)
            LAUNCH(Q35_FAM_GDN, launch_gdn_chunked(gp, st));
        else
            LAUNCH(Q35_FAM_GDN, launch_gdn_step(gp, st));
    }
    if (fused) {
        LAUNCH(Q35_FAM_OUT_PROJ, launch_linear_resid_rows(e->mix, L.out_w, e->resid, rows, 2048, pf ? L.gu_w : nullptr, gu_bytes, st));
        LAUNCH(Q35_FAM_MLP_GATEUP, launch_linear_norm_rows(e->resid, L.post_norm, L.gu_w, e->act, rows, 2 * kFF, EPI_SWIGLU,
                                                           pf ? L.down_w : nullptr, down_bytes, st));
        LAUNCH(Q35_FAM_MLP_DOWN, launch_linear_resid_rows(e->act, L.down_w, e->resid, rows, kFF, pf ? next_w : nullptr, next_w_bytes, st));
        return Q35_OK;
    }
    {
        const int sp = linear_tc_splits(rows, kHidden, 2048, kSplitMaxRows);
        if (sp > 1) {
            LAUNCH(Q35_FAM_OUT_PROJ, launch_linear_tc_split(e->mix, L.out_w, e->split_ws, rows, kHidden, 2048, sp, e->dev_status, st));
            LAUNCH(Q35_FAM_GLUE, launch_add_norm(e->resid, nullptr, nullptr, 0, nullptr, L.post_norm, e->resid, e->normed, rows, st, e->split_ws, sp));
        } else {
            LAUNCH(Q35_FAM_OUT_PROJ, launch_linear(e->mix, L.out_w, e->delta, rows, kHidden, 2048, EPI_PLAIN, nullptr, nullptr, nullptr, st, e->dev_status));
            LAUNCH(Q35_FAM_GLUE, launch_add_norm(e->resid, nullptr, nullptr, 0, e->delta, L.post_norm, e->resid, e->normed, rows, st));
        }
    }
    LAUNCH(Q35_FAM_MLP_GATEUP, launch_linear(e->normed, L.gu_w, e->act, rows, 2 * kFF, kHidden, EPI_SWIGLU, nullptr, nullptr, nullptr, st, e->dev_status));
    {
        const int sp = linear_tc_splits(rows, kHidden, kFF, kSplitMaxRows);
        if (sp > 1) {
            LAUNCH(Q35_FAM_MLP_DOWN, launch_linear_tc_split(e->act, L.down_w, e->split_ws, rows, kHidden, kFF, sp, e->dev_status, st));
            LAUNCH(Q35_FAM_GLUE, launch_add_norm(e->resid, nullptr, nullptr, 0, nullptr, next_norm, e->resid, e->normed, rows, st, e->split_ws, sp));
        } else {
            LAUNCH(Q35_FAM_MLP_DOWN, launch_linear(e->act, L.down_w, e->delta, rows, kHidden, kFF, EPI_PLAIN, nullptr, nullptr, nullptr, st, e->dev_status));
            LAUNCH(Q35_FAM_GLUE, launch_add_norm(e->resid, nullptr, nullptr, 0, e->delta, next_norm, e->resid, e->normed, rows, st));
        }
    }
    return Q35_OK;
}

// ids: compact [lanes*T].  Leaves the final-normed rows in e->normed [lanes*T][1024].
static int run_body(q35_engine* e, q35_state* s, const int* ids, int T, int checkpoint, cudaStream_t st) {
    const int rows = s->lanes * T;
    REQUIRE(rows <= e->max_rows, Q35_ERR_CAPACITY, "body of %d rows exceeds engine max_rows %d", rows, e->max_rows);
    REQUIRE(s->host_pos_hi + T <= s->max_ctx, Q35_ERR_CAPACITY, "position %d + %d beyond max_ctx %d", s->host_pos_hi, T, s->max_ctx);
    pdl_set_rows(rows);
    const bool fused = body_fused(e, rows);
    LAUNCH(Q35_FAM_GLUE, launch_add_norm(nullptr, ids, e->embed, e->vocab, nullptr, e->layers[0].input_norm,
                                         e->resid, e->normed, rows, st));
    for (int l = 0; l < kLayers; ++l) {
        const uint16_t* next_norm = (l + 1 < kLayers) ? e->layers[l + 1].input_norm : e->final_norm;
        // what the last projection of the block pulls into L2: the next block's in-projection, or (last block) the
        // first part of the tied head's table
        const void* next_w = (l + 1 < kLayers) ? (const void*)e->layers[l + 1].in_w : (const void*)e->embed;
        size_t next_bytes = (l + 1 < kLayers) ? (size_t)e->layers[l + 1].in_n * kHidden * 2 : (size_t)e->vocab * kHidden * 2;
        if (next_bytes > ((size_t)48 << 20)) next_bytes = (size_t)48 << 20;
        int rc = run_layer(e, s, l, T, checkpoint, fused, !fused || l == 0, next_norm, next_w, next_bytes, st);
        if (rc != Q35_OK) return rc;
    }
    if (fused)      // the head, the drafts and the caller read plain normed rows
        LAUNCH(Q35_FAM_GLUE, launch_add_norm(e->resid, nullptr, nullptr, 0, nullptr, e->final_norm, nullptr, e->normed, rows, st));
    return Q35_OK;
}

// tied head + device argmax over `rows` rows of x
static int run_head(q35_engine* e, const uint16_t* x, int rows, int* tokens, float* logits, cudaStream_t st) {
    REQUIRE(rows <= e->head_rows_cap, Q35_ERR_CAPACITY, "head over %d rows exceeds the engine's %d head rows", rows, e->head_rows_cap);
    int n_parts = linear_argmax_parts(rows, e->vocab);
    REQUIRE(n_parts <= e->parts_cap, Q35_ERR_CAPACITY, "argmax partials overflow");
    LAUNCH(Q35_FAM_HEAD, launch_linear(x, e->embed, nullptr, rows, e->vocab, kHidden, EPI_ARGMAX, e->partials, logits, &n_parts, st, e->dev_status));
    LAUNCH(Q35_FAM_HEAD, launch_argmax_final(e->partials, n_parts, rows, tokens, nullptr, st));
    return Q35_OK;
}

extern "C" int q35_decode_step(q35_engine* e, q35_state* s, const int* in_tok, int* out_tok,
                               float* logits_f32, uint16_t* normed, void* stream) {
    REQUIRE(e && s && in_tok && out_tok, Q35_ERR_ARG, "q35_decode_step: null argument");
    REQUIRE(s->e == e, Q35_ERR_STATE, "q35_decode_step: state belongs to another engine");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    int rc = run_body(e, s, in_tok, 1, 0, st);
    if (rc != Q35_OK) return rc;
    rc = run_head(e, e->normed, s->lanes, out_tok, logits_f32, st);
    if (rc != Q35_OK) return rc;
    if (normed) CK(copy_rows(normed, e->normed, (size_t)s->lanes * kHidden, st));
    LAUNCH_PLAIN(launch_add_int(s->pos, 1, s->lanes, st));
    s->host_pos_hi += 1;
    return Q35_OK;
}

extern "C" int q35_prefill(q35_engine* e, q35_state* s, const int* ids, int T, int* y0,
                           uint16_t* normed_last, void* stream) {
    REQUIRE(e && s && ids && y0, Q35_ERR_ARG, "q35_prefill: null argument");
    REQUIRE(s->e == e, Q35_ERR_STATE, "q35_prefill: state belongs to another engine");
    REQUIRE(T >= 1, Q35_ERR_ARG, "q35_prefill: T = %d", T);
    REQUIRE(s->host_pos_hi + T <= s->max_ctx, Q35_ERR_CAPACITY, "prompt of %d tokens at position %d beyond max_ctx %d", T, s->host_pos_hi, s->max_ctx);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    int Tc = e->max_rows / s->lanes;
    if (Tc > T) Tc = T;
    REQUIRE(Tc >= 1, Q35_ERR_CAPACITY, "q35_prefill: lanes exceed max_rows");
    for (int t0 = 0; t0 < T; t0 += Tc) {
        const int tc = (T - t0) < Tc ? (T - t0) : Tc;
        const int rows = s->lanes * tc;
        slice_ids_kernel<<<(rows + 255) / 256, 256, 0, st>>>(ids, T, t0, tc, e->tok2, rows);
        CK(cudaGetLastError());
        int rc = run_body(e, s, e->tok2, tc, 0, st);
        if (rc != Q35_OK) return rc;
        LAUNCH_PLAIN(launch_add_int(s->pos, tc, s->lanes, st));
        e->n_launch += 1;                         // the id-slicing kernel ahead of the body
        s->host_pos_hi += tc;
        if (t0 + tc >= T) {
            // last row of every lane -> compact [lanes][1024]
            CK(cudaMemcpy2DAsync(e->last_normed, kHidden * sizeof(uint16_t),
                                 e->normed + (size_t)(tc - 1) * kHidden, (size_t)tc * kHidden * sizeof(uint16_t),
                                 kHidden * sizeof(uint16_t), s->lanes, cudaMemcpyDeviceToDevice, st));
        }
    }
    int rc = run_head(e, e->last_normed, s->lanes, y0, nullptr, st);
    if (rc != Q35_OK) return rc;
    if (normed_last) CK(copy_rows(normed_last, e->last_normed, (size_t)s->lanes * kHidden, st));
    return Q35_OK;
}

// ------------------------------------------------------------------------------------------------
// MTP
// ------------------------------------------------------------------------------------------------
extern "C" int q35_mtp_state_reset(q35_mtp_state* m, void* stream) {
    REQUIRE(m, Q35_ERR_ARG, "q35_mtp_state_reset: null state");
    CK(cudaMemsetAsync(m->n, 0, m->lanes * sizeof(int), static_cast<cudaStream_t>(stream)));
    m->host_n_hi = 0;
    m->drafts_pending = 0;
    return Q35_OK;
}

// The same for the draft cache: a round that does not accept everything drops its k rows on the
// device, while the host's bound only ever grows.
extern "C" int q35_mtp_state_sync_bound(q35_mtp_state* m, void* stream) {
    REQUIRE(m, Q35_ERR_ARG, "q35_mtp_state_sync_bound: null state");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    std::vector<int> n(m->lanes);
    CK(cudaMemcpyAsync(n.data(), m->n, m->lanes * sizeof(int), cudaMemcpyDeviceToHost, st));
    CK(cudaStreamSynchronize(st));
    int hi = 0;
    for (int v : n) hi = v > hi ? v : hi;
    m->host_n_hi = hi;
    return Q35_OK;
}

// A caller that replays a captured CUDA graph of a speculative round reports the rows its drafts
// append (the captured call counted once), like q35_state_note_advance for the positions.
extern "C" int q35_mtp_state_note_advance(q35_mtp_state* m, int n) {
    REQUIRE(m, Q35_ERR_ARG, "q35_mtp_state_note_advance: null state");
    REQUIRE(m->host_n_hi + n <= m->max_ctx && m->host_n_hi + n >= 0, Q35_ERR_CAPACITY,
            "draft cache rows %d + %d beyond %d", m->host_n_hi, n, m->max_ctx);
    m->host_n_hi += n;
    return Q35_OK;
}

extern "C" int q35_mtp_state_create(q35_engine* e, q35_state* s, int max_ctx, q35_mtp_state** out) {
    REQUIRE(e && s && out, Q35_ERR_ARG, "q35_mtp_state_create: null argument");
    REQUIRE(e->has_mtp, Q35_ERR_STATE, "engine was created without MTP weights");
    REQUIRE(s->e == e, Q35_ERR_STATE, "state belongs to another engine");
    REQUIRE(2 * s->lanes <= e->head_rows_cap, Q35_ERR_CAPACITY, "verify needs 2 * lanes <= %d head rows", e->head_rows_cap);
    REQUIRE(max_ctx >= 1 && max_ctx <= 8192, Q35_ERR_CAPACITY, "max_ctx %d out of range", max_ctx);
    q35_mtp_state* m = new q35_mtp_state();
    m->e = e; m->s = s; m->lanes = s->lanes; m->max_ctx = max_ctx;
    m->pages_per_lane = (max_ctx + kKvPage - 1) / kKvPage;
    const size_t n_pages = (size_t)m->lanes * m->pages_per_lane;
    const size_t sn = (size_t)kGdnLayers * s->lanes * kGdnHeads * kDk * kDv;
    const size_t wn = (size_t)kGdnLayers * s->lanes * 3 * kConvCh;
    cudaError_t ce = cudaSuccess;
    if (ce == cudaSuccess) ce = dev_alloc(m->allocs, &m->kpool, n_pages * kPageElems);
    if (ce == cudaSuccess) ce = dev_alloc(m->allocs, &m->vpool, n_pages * kPageElems);
    if (ce == cudaSuccess) ce = dev_alloc(m->allocs, &m->table, n_pages);
    if (ce == cudaSuccess) ce = dev_alloc(m->allocs, &m->n, (size_t)m->lanes);
    m->n_pages = (long long)n_pages;
    if (ce == cudaSuccess && (!attn_make_pool_map(m->kmap, m->kpool, m->n_pages) ||
                              !attn_make_pool_map(m->vmap, m->vpool, m->n_pages)))
        ce = cudaErrorInvalidValue;
    // shadow state buffers + per-lane selector, owned by the target state from now on
    if (ce == cudaSuccess && !s->S[1]) {
        ce = dev_alloc(s->allocs, &s->S[1], sn);
        if (ce == cudaSuccess) ce = dev_alloc(s->allocs, &s->win[1], wn);
        if (ce == cudaSuccess) ce = dev_alloc(s->allocs, &s->sel, (size_t)s->lanes);
        if (ce == cudaSuccess) ce = cudaMemset(s->S[1], 0, sn * sizeof(float));
        if (ce == cudaSuccess) ce = cudaMemset(s->win[1], 0, wn * sizeof(uint16_t));
        if (ce == cudaSuccess) ce = cudaMemset(s->sel, 0, s->lanes * sizeof(int));
    }
    if (ce == cudaSuccess) {
        std::vector<int> t(n_pages);
        for (size_t i = 0; i < n_pages; ++i) t[i] = (int)i;
        ce = cudaMemcpy(m->table, t.data(), n_pages * sizeof(int), cudaMemcpyHostToDevice);
    }
    if (ce == cudaSuccess) ce = cudaMemset(m->n, 0, m->lanes * sizeof(int));
    if (ce == cudaSuccess) ce = cudaDeviceSynchronize();
    if (ce != cudaSuccess) {
        int rc = fail(Q35_ERR_CUDA, "q35_mtp_state_create: %s", cudaGetErrorString(ce));
        free_all(m->allocs);
        delete m;
        return rc;
    }
    *out = m;
    return Q35_OK;
}

extern "C" int q35_mtp_state_destroy(q35_mtp_state* m) {
    if (!m) return Q35_OK;
    free_all(m->allocs);
    delete m;
    return Q35_OK;
}

// One draft pass of the MTP block for every lane (speccheck/mtp.py:57-83): proposal ids, the
// block's output hidden in e->normed, one row appended to the draft cache.
static int draft_once(q35_engine* e, q35_mtp_state* m, const uint16_t* h_norm, const int* y_next,
                      const int* pos, int* proposal, cudaStream_t st, uint16_t* u_out = nullptr,
                      float* logits_out = nullptr) {
    const int rows = m->lanes;
    const PackedLayer& L = e->mtp_layer;
    // pair = [ N(E[y]; norm_emb) | N(h; norm_hid) ], written as two 1024-wide halves of [rows][2048]
    CK(launch_add_norm(nullptr, y_next, e->embed, e->vocab, nullptr, e->mtp_norm_emb, nullptr, e->normed, rows, st));
    CK(launch_add_norm(h_norm, nullptr, nullptr, 0, nullptr, e->mtp_norm_hid, nullptr, e->delta, rows, st));
    CK(cudaMemcpy2DAsync(e->pair, 2048 * sizeof(uint16_t), e->normed, kHidden * sizeof(uint16_t),
                         kHidden * sizeof(uint16_t), rows, cudaMemcpyDeviceToDevice, st));
    CK(cudaMemcpy2DAsync(e->pair + kHidden, 2048 * sizeof(uint16_t), e->delta, kHidden * sizeof(uint16_t),
                         kHidden * sizeof(uint16_t), rows, cudaMemcpyDeviceToDevice, st));
    CK(launch_linear(e->pair, e->mtp_fc, e->resid, rows, kHidden, 2048, EPI_PLAIN, nullptr, nullptr, nullptr, st, e->dev_status));
    if (u_out) CK(copy_rows(u_out, e->resid, (size_t)rows * kHidden, st));
    CK(launch_add_norm(e->resid, nullptr, nullptr, 0, nullptr, L.input_norm, nullptr, e->normed, rows, st));
    CK(launch_linear(e->normed, L.in_w, e->proj, rows, L.in_n, kHidden, EPI_PLAIN, nullptr, nullptr, nullptr, st, e->dev_status));
    AttnParams ap{};
    ap.proj = e->proj; ap.q_norm = L.q_norm; ap.k_norm = L.k_norm;
    ap.kpool = m->kpool; ap.vpool = m->vpool; ap.page_table = m->table;
    ap.pages_per_lane = m->pages_per_lane; ap.table_lane_stride = m->pages_per_lane;
    ap.slot = m->n; ap.rope_pos = pos; ap.inv_freq = e->inv_freq;
    ap.out = e->mix; ap.lanes = rows; ap.T = 1; ap.max_ctx = m->max_ctx;
    ap.n_pages = m->n_pages; ap.kmap = m->kmap; ap.vmap = m->vmap; ap.status = e->dev_status;
    CK(launch_attn(ap, st));
    CK(launch_linear(e->mix, L.out_w, e->delta, rows, kHidden, 2048, EPI_PLAIN, nullptr, nullptr, nullptr, st, e->dev_status));
    CK(launch_add_norm(e->resid, nullptr, nullptr, 0, e->delta, L.post_norm, e->resid, e->normed, rows, st));
    CK(launch_linear(e->normed, L.gu_w, e->act, rows, 2 * kFF, kHidden, EPI_SWIGLU, nullptr, nullptr, nullptr, st, e->dev_status));
    CK(launch_linear(e->act, L.down_w, e->delta, rows, kHidden, kFF, EPI_PLAIN, nullptr, nullptr, nullptr, st, e->dev_status));
    CK(launch_add_norm(e->resid, nullptr, nullptr, 0, e->delta, e->mtp_norm_out, e->resid, e->normed, rows, st));
    int rc = run_head(e, e->normed, rows, proposal, logits_out, st);
    if (rc != Q35_OK) return rc;
    LAUNCH_PLAIN(launch_add_int(m->n, 1, rows, st));
    e->n_launch += 11;                            // the block's kernels above (two norms, five projections, attention, two add + norms, fc)
    m->host_n_hi += 1;
    m->drafts_pending += 1;
    return Q35_OK;
}

// The same draft with the block's intermediate rows copied out, for stage-level parity against the
// reference's taps (speccheck/mtp.py:57-83: `mtp.u`, `mtp.x_d`, `mtp.logits_last`).
extern "C" int q35_mtp_draft_taps(q35_engine* e, q35_mtp_state* m, const uint16_t* h_norm, const int* y_next,
                                  const int* pos, int* proposal, uint16_t* u_out, uint16_t* xd_out,
                                  float* logits_out, void* stream) {
    REQUIRE(e && m && h_norm && y_next && pos && proposal, Q35_ERR_ARG, "q35_mtp_draft_taps: null argument");
    REQUIRE(m->e == e, Q35_ERR_STATE, "q35_mtp_draft_taps: state belongs to another engine");
    REQUIRE(m->host_n_hi + 1 <= m->max_ctx, Q35_ERR_CAPACITY, "draft cache full (%d rows)", m->max_ctx);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    pdl_set_rows(m->lanes);
    int rc = draft_once(e, m, h_norm, y_next, pos, proposal, st, u_out, logits_out);
    if (rc != Q35_OK) return rc;
    if (xd_out) CK(copy_rows(xd_out, e->normed, (size_t)m->lanes * kHidden, st));
    return Q35_OK;
}

extern "C" int q35_mtp_draft(q35_engine* e, q35_mtp_state* m, const uint16_t* h_norm, const int* y_next,
                             const int* pos, int* proposal, void* stream) {
    REQUIRE(e && m && h_norm && y_next && pos && proposal, Q35_ERR_ARG, "q35_mtp_draft: null argument");
    REQUIRE(m->e == e, Q35_ERR_STATE, "q35_mtp_draft: state belongs to another engine");
    REQUIRE(m->host_n_hi + 1 <= m->max_ctx, Q35_ERR_CAPACITY, "draft cache full (%d rows)", m->max_ctx);
    pdl_set_rows(m->lanes);
    return draft_once(e, m, h_norm, y_next, pos, proposal, static_cast<cudaStream_t>(stream));
}

extern "C" int q35_mtp_state_reserve_depth(q35_mtp_state* m, int k) {
    REQUIRE(m && m->s, Q35_ERR_ARG, "q35_mtp_state_reserve_depth: null state");
    REQUIRE(k >= 1 && k < kStateBufs, Q35_ERR_ARG, "q35_mtp_state_reserve_depth: depth %d, supported 1..%d", k, kStateBufs - 1);
    q35_state* s = m->s;
    REQUIRE((k + 1) * s->lanes <= m->e->head_rows_cap && (k + 1) * s->lanes <= m->e->max_rows, Q35_ERR_CAPACITY,
            "a depth-%d round needs %d rows, the engine holds %d", k, (k + 1) * s->lanes,
            m->e->head_rows_cap < m->e->max_rows ? m->e->head_rows_cap : m->e->max_rows);
    const size_t sn = (size_t)kGdnLayers * s->lanes * kGdnHeads * kDk * kDv;
    const size_t wn = (size_t)kGdnLayers * s->lanes * 3 * kConvCh;
    cudaError_t ce = cudaSuccess;
    for (int b = 1; b <= k && ce == cudaSuccess; ++b) {
        if (s->S[b]) continue;
        ce = dev_alloc(s->allocs, &s->S[b], sn);
        if (ce == cudaSuccess) ce = dev_alloc(s->allocs, &s->win[b], wn);
        if (ce == cudaSuccess) ce = cudaMemset(s->S[b], 0, sn * sizeof(float));
        if (ce == cudaSuccess) ce = cudaMemset(s->win[b], 0, wn * sizeof(uint16_t));
    }
    if (ce == cudaSuccess && !m->h_tmp) {
        ce = dev_alloc(m->allocs, &m->h_tmp, (size_t)m->lanes * kHidden);
        if (ce == cudaSuccess) ce = dev_alloc(m->allocs, &m->pos_tmp, (size_t)m->lanes);
        if (ce == cudaSuccess) ce = dev_alloc(m->allocs, &m->prop_tmp, (size_t)m->lanes);
    }
    if (ce == cudaSuccess) ce = cudaDeviceSynchronize();
    if (ce != cudaSuccess) return fail(Q35_ERR_CUDA, "q35_mtp_state_reserve_depth: %s", cudaGetErrorString(ce));
    if (k > m->depth) m->depth = k;
    return Q35_OK;
}

// k chained drafts (speccheck/mtp.py:148-153): draft j reads the hidden the block produced for
// draft j - 1 and the token draft j - 1 proposed, at position pos + j.
extern "C" int q35_mtp_draft_k(q35_engine* e, q35_mtp_state* m, const uint16_t* h_norm, const int* y_next,
                               const int* pos, int k, int* proposals, void* stream) {
    REQUIRE(e && m && h_norm && y_next && pos && proposals, Q35_ERR_ARG, "q35_mtp_draft_k: null argument");
    REQUIRE(m->e == e, Q35_ERR_STATE, "q35_mtp_draft_k: state belongs to another engine");
    REQUIRE(k >= 1 && k <= m->depth && m->h_tmp, Q35_ERR_STATE, "q35_mtp_draft_k: depth %d not reserved (q35_mtp_state_reserve_depth)", k);
    REQUIRE(m->host_n_hi + k <= m->max_ctx, Q35_ERR_CAPACITY, "draft cache full (%d rows)", m->max_ctx);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int L = m->lanes;
    pdl_set_rows(L);
    const uint16_t* h = h_norm;
    const int* y = y_next;
    const int* p = pos;
    for (int j = 0; j < k; ++j) {
        int rc = draft_once(e, m, h, y, p, m->prop_tmp, st);
        if (rc != Q35_OK) return rc;
        CK(launch_k(scatter_col_kernel, dim3((L + 255) / 256), dim3(256), 0, st, m->prop_tmp, proposals, k, j, L));
        if (j + 1 < k) {
            CK(copy_rows(m->h_tmp, e->normed, (size_t)L * kHidden, st));
            CK(launch_k(add_const_kernel, dim3((L + 255) / 256), dim3(256), 0, st, pos, j + 1, m->pos_tmp, L));
            // prop_tmp is read by the next pass's first kernel and rewritten by its last: stream order suffices
            h = m->h_tmp; y = m->prop_tmp; p = m->pos_tmp;
        }
    }
    return Q35_OK;
}

static int verify_round(q35_engine* e, q35_state* s, q35_mtp_state* m, const int* cur, const int* cand, int k,
                        int* emit, int* n_emit, uint16_t* h_next, cudaStream_t st) {
    const int L = s->lanes;
    // a rejecting round drops k rows from the draft cache: they must have been drafted since the last round
    REQUIRE(m->drafts_pending >= k, Q35_ERR_STATE, "verify of depth %d after %d draft(s): draft first (q35_mtp_draft / q35_mtp_draft_k)", k, m->drafts_pending);
    m->drafts_pending = 0;
    CK(launch_k(verify_ids_kernel, dim3((L * (k + 1) + 255) / 256), dim3(256), 0, st, cur, cand, k, e->tok2, L));
    int rc = run_body(e, s, e->tok2, k + 1, k, st);
    if (rc != Q35_OK) return rc;
    rc = run_head(e, e->normed, (k + 1) * L, e->tgt, nullptr, st);
    if (rc != Q35_OK) return rc;
    CK(launch_k(mtp_verdict_kernel, dim3((L + 7) / 8), dim3(256), 0, st, cand, e->tgt, e->normed, k, emit, n_emit, h_next,
                s->pos, s->sel, m->n, L));
    e->n_launch += 2;                             // the id-gather ahead of the body and the verdict
    s->host_pos_hi += k + 1;   // upper bound: lanes that rejected sit lower
    return Q35_OK;
}

extern "C" int q35_mtp_verify(q35_engine* e, q35_state* s, q35_mtp_state* m, const int* cur,
                              const int* cand, int* emit, int* n_emit, uint16_t* h_next, void* stream) {
    REQUIRE(e && s && m && cur && cand && emit && n_emit && h_next, Q35_ERR_ARG, "q35_mtp_verify: null argument");
    REQUIRE(m->s == s && s->e == e && s->S[1] && s->sel, Q35_ERR_STATE, "q35_mtp_verify: MTP state not attached to this state");
    return verify_round(e, s, m, cur, cand, 1, emit, n_emit, h_next, static_cast<cudaStream_t>(stream));
}

extern "C" int q35_mtp_verify_k(q35_engine* e, q35_state* s, q35_mtp_state* m, const int* cur,
                                const int* cands, int k, int* emit, int* n_emit, uint16_t* h_next, void* stream) {
    REQUIRE(e && s && m && cur && cands && emit && n_emit && h_next, Q35_ERR_ARG, "q35_mtp_verify_k: null argument");
    REQUIRE(m->s == s && s->e == e && s->sel, Q35_ERR_STATE, "q35_mtp_verify_k: MTP state not attached to this state");
    REQUIRE(k >= 1 && k <= m->depth && s->S[k], Q35_ERR_STATE, "q35_mtp_verify_k: depth %d not reserved (q35_mtp_state_reserve_depth)", k);
    return verify_round(e, s, m, cur, cands, k, emit, n_emit, h_next, static_cast<cudaStream_t>(stream));
}

// ------------------------------------------------------------------------------------------------
// single stages
// ------------------------------------------------------------------------------------------------
extern "C" const char* q35_op_linear_route(int rows, int N, int K, int epilogue) {
    return linear_route(rows, N, K, epilogue == 1 ? EPI_SWIGLU : (epilogue == 2 ? EPI_ARGMAX : EPI_PLAIN));
}

extern "C" int q35_engine_launch_count(q35_engine* e, long long* count_host) {
    REQUIRE(e && count_host, Q35_ERR_ARG, "q35_engine_launch_count: null argument");
    *count_host = e->n_launch;
    return Q35_OK;
}

extern "C" int q35_engine_clear_status(q35_engine* e, void* stream) {
    REQUIRE(e, Q35_ERR_ARG, "q35_engine_clear_status: null engine");
    CK(cudaMemsetAsync(e->dev_status, 0, sizeof(int), static_cast<cudaStream_t>(stream)));
    return Q35_OK;
}

extern "C" int q35_op_linear_resid(q35_engine* e, const uint16_t* x, const uint16_t* W, uint16_t* resid, int rows,
                                   int K, void* stream) {
    REQUIRE(e && x && W && resid, Q35_ERR_ARG, "q35_op_linear_resid: null argument");
    REQUIRE(rows >= 1 && rows <= kFusedMaxRows, Q35_ERR_CAPACITY, "q35_op_linear_resid: rows = %d, supported 1..%d", rows, kFusedMaxRows);
    REQUIRE(K == 2048 || K == 3584, Q35_ERR_ARG, "q35_op_linear_resid: K = %d unsupported", K);
    REQUIRE(aligned16(x) && aligned16(W) && aligned16(resid), Q35_ERR_ARG, "q35_op_linear_resid: pointers must be 16-byte aligned");
    pdl_set_rows(rows);
    CK(launch_linear_resid_rows(x, W, resid, rows, K, nullptr, 0, static_cast<cudaStream_t>(stream)));
    return Q35_OK;
}

extern "C" int q35_op_linear_norm(q35_engine* e, const uint16_t* resid, const uint16_t* nw, const uint16_t* W,
                                  uint16_t* out, int rows, int N, int swiglu, void* stream) {
    REQUIRE(e && resid && nw && W && out, Q35_ERR_ARG, "q35_op_linear_norm: null argument");
    REQUIRE(rows >= 1 && rows <= kFusedMaxRows, Q35_ERR_CAPACITY, "q35_op_linear_norm: rows = %d, supported 1..%d", rows, kFusedMaxRows);
    REQUIRE(N >= 8 && N % 8 == 0, Q35_ERR_ARG, "q35_op_linear_norm: N = %d must be a multiple of 8", N);
    REQUIRE(aligned16(resid) && aligned16(W) && aligned16(out) && aligned16(nw), Q35_ERR_ARG, "q35_op_linear_norm: pointers must be 16-byte aligned");
    pdl_set_rows(rows);
    CK(launch_linear_norm_rows(resid, nw, W, out, rows, N, swiglu ? EPI_SWIGLU : EPI_PLAIN, nullptr, 0,
                               static_cast<cudaStream_t>(stream)));
    return Q35_OK;
}

// The output / down projection stage exactly as a body runs it: resid <- bf16(resid + bf16(x . W^T)) and, above
// 16 rows, normed = N(resid; nw) by the add + norm kernel (at most 16 rows: the next projection applies the norm).
extern "C" int q35_op_proj_residual(q35_engine* e, const uint16_t* x, const uint16_t* W, uint16_t* resid,
                                    const uint16_t* nw, uint16_t* normed, int rows, int K, void* stream) {
    REQUIRE(e && x && W && resid && nw && normed, Q35_ERR_ARG, "q35_op_proj_residual: null argument");
    REQUIRE(rows >= 1 && rows <= e->max_rows, Q35_ERR_CAPACITY, "q35_op_proj_residual: rows = %d, the engine holds %d", rows, e->max_rows);
    REQUIRE(K == 2048 || K == 3584, Q35_ERR_ARG, "q35_op_proj_residual: K = %d unsupported", K);
    REQUIRE(aligned16(x) && aligned16(W) && aligned16(resid) && aligned16(nw) && aligned16(normed), Q35_ERR_ARG,
            "q35_op_proj_residual: pointers must be 16-byte aligned");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    pdl_set_rows(rows);
    if (body_fused(e, rows)) {
        CK(launch_linear_resid_rows(x, W, resid, rows, K, nullptr, 0, st));
        return Q35_OK;
    }
    const int sp = linear_tc_splits(rows, kHidden, K, kSplitMaxRows);
    if (sp > 1) {
        CK(launch_linear_tc_split(x, W, e->split_ws, rows, kHidden, K, sp, e->dev_status, st));
        CK(launch_add_norm(resid, nullptr, nullptr, 0, nullptr, nw, resid, normed, rows, st, e->split_ws, sp));
    } else {
        CK(launch_linear(x, W, e->delta, rows, kHidden, K, EPI_PLAIN, nullptr, nullptr, nullptr, st, e->dev_status));
        CK(launch_add_norm(resid, nullptr, nullptr, 0, e->delta, nw, resid, normed, rows, st));
    }
    return Q35_OK;
}
extern "C" const char* q35_op_proj_residual_route(q35_engine* e, int rows, int K) {
    if (e == nullptr) return "unsupported";
    if (body_fused(e, rows)) return "gemv_rows_kernel (residual epilogue)";
    if (linear_tc_splits(rows, kHidden, K, kSplitMaxRows) > 1) return "gemm_tc_kernel<128,4> split-K + add_norm_split_kernel";
    static thread_local char buf[160];
    snprintf(buf, sizeof(buf), "%s + add_norm_kernel", linear_route(rows, kHidden, K, EPI_PLAIN));
    return buf;
}

// One block of the decoder in isolation, for layer-level teacher forcing: x_in [lanes*T][1024] are the
// block's input residual rows, x_out receives its output rows; the lanes' state is read at their current
// positions and updated (state of that layer, one KV row), the positions are NOT advanced.
extern "C" int q35_op_layer(q35_engine* e, q35_state* s, int layer, const uint16_t* x_in, uint16_t* x_out, int T,
                            int fused, void* stream) {
    REQUIRE(e && s && x_in && x_out, Q35_ERR_ARG, "q35_op_layer: null argument");
    REQUIRE(s->e == e, Q35_ERR_STATE, "q35_op_layer: state belongs to another engine");
    REQUIRE(layer >= 0 && layer < kLayers && T >= 1, Q35_ERR_ARG, "q35_op_layer: layer %d, T %d", layer, T);
    const int rows = s->lanes * T;
    REQUIRE(rows <= e->max_rows, Q35_ERR_CAPACITY, "body of %d rows exceeds engine max_rows %d", rows, e->max_rows);
    REQUIRE(s->host_pos_hi + T <= s->max_ctx, Q35_ERR_CAPACITY, "position %d + %d beyond max_ctx %d", s->host_pos_hi, T, s->max_ctx);
    const bool use_fused = fused < 0 ? body_fused(e, rows) : (fused != 0 && rows <= kFusedMaxRows);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    pdl_set_rows(rows);
    CK(launch_add_norm(x_in, nullptr, nullptr, 0, nullptr, e->layers[layer].input_norm, e->resid, e->normed, rows, st));
    const uint16_t* next_norm = (layer + 1 < kLayers) ? e->layers[layer + 1].input_norm : e->final_norm;
    int rc = run_layer(e, s, layer, T, 0, use_fused, true, next_norm, nullptr, 0, st);
    if (rc != Q35_OK) return rc;
    CK(copy_rows(x_out, e->resid, (size_t)rows * kHidden, st));
    return Q35_OK;
}

extern "C" int q35_op_add_norm(const uint16_t* x, const uint16_t* delta, const uint16_t* w,
                               uint16_t* sum_out, uint16_t* normed_out, int rows, void* stream) {
    REQUIRE(x && w && rows >= 1, Q35_ERR_ARG, "q35_op_add_norm: bad argument");
    REQUIRE(aligned16(x) && aligned16(w) && aligned16(delta) && aligned16(sum_out) && aligned16(normed_out),
            Q35_ERR_ARG, "q35_op_add_norm: pointers must be 16-byte aligned");
    CK(launch_add_norm(x, nullptr, nullptr, 0, delta, w, sum_out, normed_out, rows, static_cast<cudaStream_t>(stream)));
    return Q35_OK;
}

// The stage entry points that take no engine report a bounded wait that ran out through this word of the
// library image (one per device that loads the library); q35_ops_status reads and clears it.
static __device__ int g_ops_status;
static int* ops_status_ptr() {
    static int* ptr[kMaxDevices] = {nullptr};        // every writer stores the same address
    const int dev = current_device_slot();
    if (dev < 0) return nullptr;
    if (ptr[dev] == nullptr) {
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, g_ops_status) != cudaSuccess) return nullptr;
        ptr[dev] = static_cast<int*>(p);
    }
    return ptr[dev];
}

extern "C" int q35_ops_status(int* status_host) {
    REQUIRE(status_host, Q35_ERR_ARG, "q35_ops_status: null argument");
    int* d = ops_status_ptr();
    REQUIRE(d != nullptr, Q35_ERR_CUDA, "q35_ops_status: no current device");
    CK(cudaDeviceSynchronize());
    CK(cudaMemcpy(status_host, d, sizeof(int), cudaMemcpyDeviceToHost));
    if (*status_host != 0) CK(cudaMemset(d, 0, sizeof(int)));
    return Q35_OK;
}

extern "C" int q35_op_linear(const uint16_t* x, const uint16_t* W, uint16_t* out, int rows, int N, int K,
                             void* stream) {
    REQUIRE(x && W && out && rows >= 1, Q35_ERR_ARG, "q35_op_linear: bad argument");
    REQUIRE(N >= 8 && N % 8 == 0, Q35_ERR_ARG, "q35_op_linear: N = %d must be a multiple of 8", N);
    REQUIRE(K == 1024 || K == 2048 || K == 3584, Q35_ERR_ARG, "q35_op_linear: K = %d unsupported", K);
    REQUIRE(aligned16(x) && aligned16(W) && aligned16(out), Q35_ERR_ARG, "q35_op_linear: pointers must be 16-byte aligned");
    pdl_set_rows(rows);
    CK(launch_linear(x, W, out, rows, N, K, EPI_PLAIN, nullptr, nullptr, nullptr, static_cast<cudaStream_t>(stream), ops_status_ptr()));
    return Q35_OK;
}

extern "C" int q35_pack_gate_up(const uint16_t* gate, const uint16_t* up, uint16_t* Wgu, void* stream) {
    REQUIRE(gate && up && Wgu && aligned16(gate) && aligned16(up) && aligned16(Wgu), Q35_ERR_ARG, "q35_pack_gate_up: bad argument");
    CK(launch_pack_gate_up(gate, up, Wgu, static_cast<cudaStream_t>(stream)));
    return Q35_OK;
}

extern "C" int q35_op_mlp_gateup(const uint16_t* x, const uint16_t* Wgu, uint16_t* act, int rows, void* stream) {
    REQUIRE(x && Wgu && act && rows >= 1 && aligned16(x) && aligned16(Wgu) && aligned16(act), Q35_ERR_ARG, "q35_op_mlp_gateup: bad argument");
    pdl_set_rows(rows);
    CK(launch_linear(x, Wgu, act, rows, 2 * kFF, kHidden, EPI_SWIGLU, nullptr, nullptr, nullptr, static_cast<cudaStream_t>(stream), ops_status_ptr()));
    return Q35_OK;
}

extern "C" int q35_op_lm_head(q35_engine* e, const uint16_t* x, int rows, int* tokens, float* logits_f32, void* stream) {
    REQUIRE(e && x && tokens && rows >= 1 && aligned16(x), Q35_ERR_ARG, "q35_op_lm_head: bad argument");
    pdl_set_rows(rows);
    return run_head(e, x, rows, tokens, logits_f32, static_cast<cudaStream_t>(stream));
}

extern "C" int q35_lm_head_argmax_static(const uint16_t* x, const uint16_t* embed, int vocab, int rows,
                                         int* tokens, void* stream) {
    REQUIRE(x && embed && tokens, Q35_ERR_ARG, "q35_lm_head_argmax_static: null argument");
    REQUIRE(aligned16(x) && aligned16(embed), Q35_ERR_ARG, "q35_lm_head_argmax_static: x / embed must be 16-byte aligned");
    REQUIRE(rows >= 1 && rows <= kStaticHeadMaxRows, Q35_ERR_CAPACITY,
            "q35_lm_head_argmax_static: rows = %d, the fixed scratch holds at most %d", rows, kStaticHeadMaxRows);
    REQUIRE(vocab >= 8 && vocab % 8 == 0 && vocab <= kStaticHeadMaxVocab, Q35_ERR_CAPACITY,
            "q35_lm_head_argmax_static: vocab = %d, must be a multiple of 8 and at most %d", vocab, kStaticHeadMaxVocab);
    CK(launch_lm_head_static(x, embed, vocab, rows, tokens, static_cast<cudaStream_t>(stream)));
    return Q35_OK;
}

extern "C" int q35_op_gdn_step(uint16_t* proj, const uint16_t* conv_w, const uint16_t* A_log,
                               const uint16_t* dt_bias, const uint16_t* norm_w, float* S, uint16_t* window,
                               uint16_t* y, int lanes, int T, void* stream) {
    REQUIRE(proj && conv_w && A_log && dt_bias && norm_w && S && window && y, Q35_ERR_ARG, "q35_op_gdn_step: null argument");
    REQUIRE(lanes >= 1 && lanes <= 65535 && T >= 1, Q35_ERR_ARG, "q35_op_gdn_step: lanes %d T %d", lanes, T);
    REQUIRE(aligned16(S) && aligned16(conv_w) && aligned16(proj) && aligned16(window), Q35_ERR_ARG,
            "q35_op_gdn_step: S / conv_w / proj / window must be 16-byte aligned");
    GdnParams gp{};
    gp.proj = proj; gp.conv_w = conv_w; gp.A_log = A_log; gp.dt_bias = dt_bias; gp.norm_w = norm_w;
    gp.S[0] = S; gp.win[0] = window; gp.sel = nullptr;      // GdnParams gp{} left the shadow buffers null
    gp.y = y; gp.lanes = lanes; gp.T = T; gp.checkpoint = 0;
    pdl_set_rows(lanes * T);
    if (T >= kGdnChunkMinT)
        CK(launch_gdn_chunked(gp, static_cast<cudaStream_t>(stream)));
    else
        CK(launch_gdn_step(gp, static_cast<cudaStream_t>(stream)));
    return Q35_OK;
}

extern "C" int q35_op_attn_decode(q35_engine* e, const uint16_t* proj, const uint16_t* q_norm,
                                  const uint16_t* k_norm, uint16_t* kpool, uint16_t* vpool,
                                  const int* page_table, int pages_per_lane, const int* ctx,
                                  uint16_t* out, int lanes, int T, void* stream) {
    REQUIRE(e && proj && q_norm && k_norm && kpool && vpool && page_table && ctx && out, Q35_ERR_ARG, "q35_op_attn_decode: null argument");
    REQUIRE(lanes >= 1 && T >= 1 && pages_per_lane >= 1 && pages_per_lane * kKvPage <= 8192, Q35_ERR_ARG, "q35_op_attn_decode: bad sizes");
    AttnParams ap{};
    ap.proj = proj; ap.q_norm = q_norm; ap.k_norm = k_norm; ap.kpool = kpool; ap.vpool = vpool;
    ap.page_table = page_table; ap.pages_per_lane = pages_per_lane; ap.table_lane_stride = pages_per_lane;
    ap.slot = ctx; ap.rope_pos = ctx; ap.inv_freq = e->inv_freq; ap.out = out; ap.lanes = lanes; ap.T = T;
    ap.max_ctx = pages_per_lane * kKvPage;
    ap.n_pages = (long long)lanes * pages_per_lane; ap.kmap = nullptr; ap.vmap = nullptr; ap.status = e->dev_status;
    CK(launch_attn(ap, static_cast<cudaStream_t>(stream)));
    return Q35_OK;
}
