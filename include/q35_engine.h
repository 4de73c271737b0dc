/*
 * C-ABI of the B200-native Qwen3.5-0.8B text-tower decode engine.
 *
 * Every entry point is `extern "C"`, takes plain pointers and sizes, returns an int status
 * (0 = ok) and never throws; q35_last_error() returns the message of the calling thread's last
 * failure.  Unless a parameter says "host", every pointer is a DEVICE pointer.  Calls only
 * enqueue work on the given CUDA stream (a cudaStream_t passed as void*); none synchronises.
 * bf16 tensors are passed as their 16-bit patterns (uint16_t), like the reference's launchers.
 *
 * "lane" = one independent request (a batch row).  The reference engine serves one request; each
 * function below is the L-lane form of the reference interface it cites (paths are relative to
 * the reference repository).
 */
#ifndef Q35_ENGINE_H
#define Q35_ENGINE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
    Q35_OK = 0,
    Q35_ERR_ARG = 1,       /* null / misaligned pointer, size out of range.  Token ids live in device
                              memory and are not read by the host: the embedding gather clamps them
                              to [0, vocab); a host-buffer caller validates them before the copy     */
    Q35_ERR_CUDA = 2,      /* a CUDA runtime call failed                                             */
    Q35_ERR_CAPACITY = 3,  /* lanes, rows or context beyond what the object was created for          */
    Q35_ERR_STATE = 4      /* call order violated (e.g. MTP verify without an MTP state)             */
};

enum {
    Q35_LAYERS = 24, Q35_GDN_LAYERS = 18, Q35_ATTN_LAYERS = 6, Q35_HIDDEN = 1024,
    Q35_FF = 3584, Q35_VOCAB = 248320, Q35_GDN_HEADS = 16, Q35_DK = 128, Q35_DV = 128,
    Q35_CONV_CH = 6144, Q35_CONV_K = 4, Q35_Q_HEADS = 8, Q35_KV_HEADS = 2, Q35_HEAD_DIM = 256,
    Q35_KV_PAGE = 64      /* KV positions per cache page */
};

/* kernel families of a body, for q35_profile_* (the reference's launch-census families,
 * engine/decode_step.cpp:39-52) */
enum {
    Q35_FAM_GLUE = 0, Q35_FAM_IN_PROJ = 1, Q35_FAM_GDN = 2, Q35_FAM_ATTN = 3, Q35_FAM_OUT_PROJ = 4,
    Q35_FAM_MLP_GATEUP = 5, Q35_FAM_MLP_DOWN = 6, Q35_FAM_HEAD = 7,
    Q35_FAMILIES = 8
};

typedef struct q35_engine q35_engine;
typedef struct q35_state q35_state;
typedef struct q35_mtp_state q35_mtp_state;

/* One decoder layer's parameters, [out,in] row-major bf16, as in the checkpoint
 * (speccheck/specimpl.py:100-127; engine/decode_step.cpp:127-177).  GDN layers fill the
 * `gdn_*` block and leave `attn_*` null; attention layers (l % 4 == 3) the reverse. */
typedef struct {
    const uint16_t* input_norm;   /* [1024]                                  */
    const uint16_t* post_norm;    /* [1024]  post_attention_layernorm        */
    const uint16_t* mlp_gate;     /* [3584,1024]                             */
    const uint16_t* mlp_up;       /* [3584,1024]                             */
    const uint16_t* mlp_down;     /* [1024,3584]                             */
    const uint16_t* gdn_in_qkv;   /* [6144,1024]                             */
    const uint16_t* gdn_in_z;     /* [2048,1024]                             */
    const uint16_t* gdn_in_b;     /* [16,1024]                               */
    const uint16_t* gdn_in_a;     /* [16,1024]                               */
    const uint16_t* gdn_conv;     /* [6144,1,4]                              */
    const uint16_t* gdn_A_log;    /* [16]                                    */
    const uint16_t* gdn_dt_bias;  /* [16]                                    */
    const uint16_t* gdn_norm;     /* [128]                                   */
    const uint16_t* gdn_out;      /* [1024,2048]                             */
    const uint16_t* attn_q;       /* [4096,1024]  per head [q 256 | gate 256] */
    const uint16_t* attn_k;       /* [512,1024]                              */
    const uint16_t* attn_v;       /* [512,1024]                              */
    const uint16_t* attn_q_norm;  /* [256]                                   */
    const uint16_t* attn_k_norm;  /* [256]                                   */
    const uint16_t* attn_o;       /* [1024,2048]                             */
} q35_layer_weights;

/* The MTP draft block's 15 tensors (engine/mtp_draft.h:115-132). */
typedef struct {
    const uint16_t* fc;           /* [1024,2048], operand order [embedding | hidden] */
    const uint16_t* norm_emb;     /* [1024] pre_fc_norm_embedding            */
    const uint16_t* norm_hid;     /* [1024] pre_fc_norm_hidden               */
    const uint16_t* norm_out;     /* [1024] mtp.norm                         */
    q35_layer_weights layer;      /* attention-layer fields + norms + mlp    */
} q35_mtp_weights;

typedef struct {
    const uint16_t* embed;        /* [vocab,1024]; also the tied lm_head (engine/loader.h:1-14).
                                     NOT copied: must stay valid for the engine's lifetime.       */
    const uint16_t* final_norm;   /* [1024]                                   */
    q35_layer_weights layers[Q35_LAYERS];
    int has_mtp;
    q35_mtp_weights mtp;
} q35_weights;

typedef struct {
    int vocab;            /* rows of `embed`; Q35_VOCAB for the real model, any multiple of 8 in tests */
    int max_rows;         /* scratch rows: lanes x tokens-per-lane a single body may carry             */
    float rope_inv_freq[32];  /* theta^(-2i/64), i = 0..31, computed by the caller in f32             */
} q35_config;

typedef struct {
    size_t gdn_state_bytes;    /* per lane: f32 [18][16][128][128]                       */
    size_t conv_window_bytes;  /* per lane, as stored (bf16 [18][3][6144])               */
    size_t kv_bytes;           /* per lane: K and V pages for max_ctx positions          */
    size_t per_token_bytes;    /* 12,288                                                 */
    size_t total_bytes;        /* all lanes                                              */
} q35_state_sizes;

typedef struct {
    long long weight_bytes;       /* read once per body                                     */
    long long lane_state_bytes;   /* per lane: GDN state read+write + conv window (f32 census) */
    long long kv_bytes_per_pos;   /* 12,288                                                 */
    long long flops_per_row;      /* matmul flops per token                                 */
    int launches_decode;          /* kernels one q35_decode_step enqueues for a body beyond the fused row
                                     limit: embedding + 24 x 7 + head, argmax, position advance          */
    int launches_decode_few_lanes;/* the same for a body of at most 16 rows: 24 x 5 blocks, the residual
                                     add + norm folded into the projections; equal to launches_decode
                                     when Q35_FUSE=0                                                     */
} q35_census;

const char* q35_last_error(void);
int q35_abi_version(void);

/* ---- engine: weights + scratch ---------------------------------------------------------------
 * Replaces WeightStore + allocate_scratch + prepare_weight_adapters
 * (engine/decode_step.h:479-480,595).  Packs the grouped in-projections and the interleaved
 * gate/up matrix into engine-owned memory; only `embed` is referenced in place. */
int q35_engine_create(const q35_config* cfg, const q35_weights* w, void* stream, q35_engine** out);
int q35_engine_destroy(q35_engine* e);
int q35_step_census(const q35_engine* e, q35_census* out);
/* Synchronises the device and reads the engine's status word: 0 = healthy; non-zero = a kernel gave
 * up a bounded wait (1 GDN tile fetch, 2-5 tcgen05 projection / head pipeline, 5-6 attention page ring,
 * 8 chunked prefill scan) and skipped its stores.  The
 * reference has no device-side waits; its nearest relative is the post-step
 * RequestState::check_invariants (engine/state.h:99). */
int q35_engine_status(q35_engine* e, int* status_host);
/* Clears the status word (enqueued on `stream`).  Once a kernel has raised it every later kernel of the
 * engine returns without work, so a caller that has dealt with the failure (state reset, lanes
 * re-prefilled) calls this to go on with the same engine.  The reference has no counterpart (no
 * device-side waits). */
int q35_engine_clear_status(q35_engine* e, void* stream);
/* Kernels enqueued through this engine since its creation (host counter; a kernel captured into a
 * CUDA graph counts once, at capture).  The launch census of the reference's stage_clock
 * (engine/decode_step.cpp:39-52) as one number. */
int q35_engine_launch_count(q35_engine* e, long long* count_host);
/* Per-family kernel timing with CUDA events on the launching stream (replaces the reference's
 * stage_clock, engine/stage_clock.h:59-67).  Between begin and end every kernel of every body is
 * bracketed by an event pair; end synchronises on the last event and returns the summed
 * milliseconds and launch counts per family (arrays of Q35_FAMILIES, host memory). */
int q35_profile_begin(q35_engine* e);
int q35_profile_end(q35_engine* e, double* ms_by_family, long long* launches_by_family);
/* ---- per-lane state tuple ----------------------------------------------------------------------
 * Replaces allocate_state / free_state / RequestState::reset / state_sizes
 * (engine/state.h:83-120) for `lanes` requests of up to `max_ctx` positions each. */
int q35_state_sizes_of(int lanes, int max_ctx, q35_state_sizes* out);
int q35_state_create(q35_engine* e, int lanes, int max_ctx, q35_state** out);
int q35_state_destroy(q35_state* s);
int q35_state_reset(q35_state* s, void* stream);
/* Copy the per-lane prefix lengths (position of the next token, engine/state.h:93) into
 * positions_out [lanes] (device). */
int q35_state_positions(q35_state* s, int* positions_out, void* stream);
/* The host keeps an upper bound of the lanes' positions for its capacity checks
 * (RequestState::check_invariants, engine/state.h:99); every body call adds its tokens to it.  A
 * captured CUDA graph runs no host code when replayed, so its caller reports each replay's steps
 * here.  n may be negative: the capture of a graph ran the body calls once on the host without
 * running a kernel, and the caller takes those steps back (n = -steps) so that every replay,
 * the first included, reports itself.  The bound never goes below 0 or beyond max_ctx
 * (Q35_ERR_CAPACITY). */
int q35_state_note_advance(q35_state* s, int n);
/* Speculative rounds advance a lane by 1..k+1 positions on the device; the host's bound moves by the
 * maximum.  This reads the true positions back (stream synchronisation) and tightens the bound. */
int q35_state_sync_bound(q35_state* s, void* stream);
/* Copy one lane's tuple out of / into the reference layouts (engine/state.h:86-92):
 * gdn_state f32 [18][16][128][128] (S[i][j], i over d_k), conv_window f32 [18][3][6144] row 0
 * oldest, kv_keys / kv_values bf16 [6][2][cap][256].  Null pointers are skipped. */
int q35_state_export_lane(q35_state* s, int lane, float* gdn_state, float* conv_window,
                          uint16_t* kv_keys, uint16_t* kv_values, int cap, void* stream);
int q35_state_import_lane(q35_state* s, int lane, const float* gdn_state, const float* conv_window,
                          const uint16_t* kv_keys, const uint16_t* kv_values, int cap,
                          int prefix_len, void* stream);

/* ---- the decode step ---------------------------------------------------------------------------
 * Replaces decode_step = submit_token_body + finish_token (engine/decode_step.h:524,575,582) for
 * every lane at once: embeds in_tok[lane], runs the 24 blocks, the final norm, the tied head and a
 * device argmax (ties to the lowest id), advances each lane's position by one.
 * out_tok [lanes] int32.  Optional outputs: logits_f32 [lanes][vocab], normed [lanes][1024] bf16. */
int q35_decode_step(q35_engine* e, q35_state* s, const int* in_tok, int* out_tok,
                    float* logits_f32, uint16_t* normed, void* stream);

/* ---- prefill -------------------------------------------------------------------------------------
 * Replaces prefill_wave (engine/prefill.h:155): consumes ids [lanes][T] (row-major), leaves the
 * state tuple and positions advanced by T, writes y0 [lanes] (argmax after the last prompt token)
 * and optionally the last final-norm row per lane, normed_last [lanes][1024] bf16. */
int q35_prefill(q35_engine* e, q35_state* s, const int* ids, int T, int* y0,
                uint16_t* normed_last, void* stream);

/* ---- MTP draft / verify ------------------------------------------------------------------------
 * q35_mtp_state_*: the draft block's own KV cache and the shadow buffers the verify round needs
 * (engine/mtp_draft.h:142-215, engine/mtp_verify.h:117-125). */
int q35_mtp_state_create(q35_engine* e, q35_state* s, int max_ctx, q35_mtp_state** out);
int q35_mtp_state_destroy(q35_mtp_state* m);
int q35_mtp_state_reset(q35_mtp_state* m, void* stream);
/* The draft cache's host bound only grows (one row per draft), while a round that does not accept
 * everything drops its rows on the device: read the true lengths back and tighten the bound. */
int q35_mtp_state_sync_bound(q35_mtp_state* m, void* stream);
/* Host bound of the draft cache for a caller that replays a captured CUDA graph of a round: n rows
 * per replay; negative n takes back what the capture itself added (see q35_state_note_advance);
 * Q35_ERR_CAPACITY when the cache would overflow or the bound would go below 0.  The
 * reference reads its verdict words back every round (engine/mtp_verify.h:117-125) and needs no
 * such bound; rounds chained on the device do. */
int q35_mtp_state_note_advance(q35_mtp_state* m, int n);
/* Replaces mtpdraft::draft_round (engine/mtp_draft.h:233): from the target's post-final-norm rows
 * h_norm [lanes][1024], the just-emitted tokens y_next [lanes] and the drafted positions
 * pos [lanes], propose proposal [lanes] and append one row to each lane's draft cache. */
int q35_mtp_draft(q35_engine* e, q35_mtp_state* m, const uint16_t* h_norm, const int* y_next,
                  const int* pos, int* proposal, void* stream);
/* Replaces mtpverify::verify_body + mtpaccept::accept_round (engine/mtp_verify.h:234,
 * engine/mtp_accept.h:248) with depth 1: feeds [cur, cand] at positions p, p+1 of every lane,
 * accepts cand iff it equals the target's argmax after cur, and leaves each lane's state at
 * p+1+accepted (reject = flip back to the checkpoint taken after `cur`, drop the draft's row).
 * emit [lanes][2], n_emit [lanes] (1 or 2), h_next [lanes][1024] = final-norm row the next draft
 * needs. */
int q35_mtp_verify(q35_engine* e, q35_state* s, q35_mtp_state* m, const int* cur, const int* cand,
                   int* emit, int* n_emit, uint16_t* h_next, void* stream);
/* A verify of depth k is refused with Q35_ERR_STATE unless k drafts were enqueued on this MTP state
 * since its last verify or reset: a rejecting round drops k rows from the draft cache. */
/* q35_mtp_draft with the block's intermediate rows copied out (each optional): u [lanes][1024] = the
 * fc output, xd [lanes][1024] = the block's final-norm rows, logits_f32 [lanes][vocab]
 * (speccheck/mtp.py:57-83, taps `mtp.u`, `mtp.x_d`, `mtp.logits_last`). */
int q35_mtp_draft_taps(q35_engine* e, q35_mtp_state* m, const uint16_t* h_norm, const int* y_next,
                       const int* pos, int* proposal, uint16_t* u, uint16_t* xd, float* logits_f32,
                       void* stream);
/* Depth-k rounds (k = 1 or 2; 2 is the reference's shipped round, engine/mtp_accept.h:87-140).
 * q35_mtp_state_reserve_depth allocates the k shadow state buffers a depth-k round checkpoints into
 * (one per body row except the last, engine/mtp_accept.h:135-140) and the chaining scratch.
 * q35_mtp_draft_k runs k chained drafts (draft j reads the block's output hidden and the proposal of
 * draft j-1, position pos + j; speccheck/mtp.py:148-153): proposals [lanes][k].
 * q35_mtp_verify_k feeds [cur, cand_1..cand_k] at positions p..p+k, accepts the LONGEST CORRECT
 * PREFIX n of the candidates (engine/mtp_accept.h:113-123), emits cand_1..cand_n then the target's
 * own token after them: emit [lanes][k+1] (unused slots -1), n_emit [lanes] = n + 1, state left
 * at p + n + 1 (n < k: the lane is pointed at the checkpoint after row n and the round's k draft
 * rows leave the draft cache, speccheck/mtp.py:163-166), h_next [lanes][1024] = final-norm row n. */
int q35_mtp_state_reserve_depth(q35_mtp_state* m, int k);
int q35_mtp_draft_k(q35_engine* e, q35_mtp_state* m, const uint16_t* h_norm, const int* y_next,
                    const int* pos, int k, int* proposals, void* stream);
int q35_mtp_verify_k(q35_engine* e, q35_state* s, q35_mtp_state* m, const int* cur, const int* cands,
                     int k, int* emit, int* n_emit, uint16_t* h_next, void* stream);

/* ---- single stages (what the per-stage parity tests and the projection/recurrence benchmark
 * slices call; each replaces one reference launcher) ------------------------------------------- */
/* glue_add_norm_rows (engine/kernels.h:45): sum = bf16(x + delta) (delta may be null),
 * normed = zero-centred RMSNorm(sum; w).  sum_out may alias x. */
int q35_op_add_norm(const uint16_t* x, const uint16_t* delta, const uint16_t* w,
                    uint16_t* sum_out, uint16_t* normed_out, int rows, void* stream);
/* proj_rows (engine/kernels.h:183-297): out [rows][N] = bf16(x [rows][K] . W[N][K]^T).
 * K in {1024, 2048, 3584}; N a multiple of 8. */
/* The stage entry points that take no engine (q35_op_linear, q35_op_mlp_gateup) report a bounded device
 * wait that ran out through a status word of the library itself: synchronises the device, reads the word
 * (0 = healthy, codes as for q35_engine_status) and clears it.  Unlike the engine's word it does not make
 * later kernels skip their work. */
int q35_ops_status(int* status_host);
int q35_op_linear(const uint16_t* x, const uint16_t* W, uint16_t* out, int rows, int N, int K,
                  void* stream);
/* The fused residual stream of bodies of at most 16 rows, as two stages (the reference's pairing of
 * residual adds with norms, engine/decode_step.h:9-15, prototype/glue/glue_kernels.h:84-128).
 * q35_op_linear_resid: resid [rows][1024] <- bf16(resid + bf16(x [rows][K] . W[1024][K]^T)) in place,
 * K in {2048, 3584}.  q35_op_linear_norm: out [rows][N] = bf16(N(resid; nw) . W[N][1024]^T) with the
 * zero-centred RMSNorm applied while the rows are staged (swiglu != 0: W is the row-interleaved
 * gate/up matrix and out is [rows][N/2]).  More than 16 rows: Q35_ERR_CAPACITY. */
int q35_op_linear_resid(q35_engine* e, const uint16_t* x, const uint16_t* W, uint16_t* resid, int rows,
                        int K, void* stream);
int q35_op_linear_norm(q35_engine* e, const uint16_t* resid, const uint16_t* nw, const uint16_t* W,
                       uint16_t* out, int rows, int N, int swiglu, void* stream);
/* The attention / GDN output projection or the MLP down projection as a body runs it, residual add
 * and the following norm included (decode_step.h:9-15: "add after mixer fused with post-attn norm, add
 * after MLP fused with the next input norm"): resid [rows][1024] updated in place; normed [rows][1024]
 * written above 16 rows (at most 16 rows the next projection applies the norm itself and normed is
 * left untouched).  q35_op_proj_residual_route names the kernels that stage takes. */
int q35_op_proj_residual(q35_engine* e, const uint16_t* x, const uint16_t* W, uint16_t* resid,
                         const uint16_t* nw, uint16_t* normed, int rows, int K, void* stream);
const char* q35_op_proj_residual_route(q35_engine* e, int rows, int K);
/* One decoder block in isolation (Forward._layer, speccheck/specimpl.py:426-451; the per-layer
 * teacher-forcing taps L{l}.s_in -> L{l}.s_out): x_in [lanes*T][1024] = the block's input residual
 * rows, x_out = its output rows.  Reads the lanes' state at their current positions and updates that
 * block's part of it; does NOT advance the positions.  fused: 1 / 0 force the fused / unfused
 * residual stream, -1 = what a body of this size takes. */
int q35_op_layer(q35_engine* e, q35_state* s, int layer, const uint16_t* x_in, uint16_t* x_out, int T,
                 int fused, void* stream);
/* Name of the kernel q35_op_linear (epilogue 0), q35_op_mlp_gateup (1) or q35_op_lm_head (2) routes a
 * shape to; a static string.  The reference routes by row count too (proj_rows vs its library GEMM,
 * engine/kernels_gemm.cpp:852-885) and prints the route in its stage census. */
const char* q35_op_linear_route(int rows, int N, int K, int epilogue);
/* mlp_gateup (engine/kernels.h:363-374): act [rows][3584] from x [rows][1024]; Wgu is the
 * row-interleaved matrix q35_pack_gate_up writes ([7168][1024]: row 2f = gate f, 2f+1 = up f). */
int q35_pack_gate_up(const uint16_t* gate, const uint16_t* up, uint16_t* Wgu, void* stream);
int q35_op_mlp_gateup(const uint16_t* x, const uint16_t* Wgu, uint16_t* act, int rows, void* stream);
/* lm_head_full + argmax (engine/kernels.h:939-945, engine/decode_step.cpp:1280): tokens [rows],
 * optional logits_f32 [rows][vocab].  Uses the engine's partial-argmax scratch. */
int q35_op_lm_head(q35_engine* e, const uint16_t* x, int rows, int* tokens, float* logits_f32,
                   void* stream);
/* Tied head + lowest-id argmax for callers that must not allocate device memory.  No counterpart
 * in the reference.  Some hosts of this library cannot call cudaMalloc at all: a plugin loaded
 * into a runtime that owns the whole device heap, or a serving loop that runs with a frozen memory
 * pool and treats any allocation on the hot path as a bug.  They cannot create a q35_engine (which
 * allocates its scratch), so this entry point takes only inputs and outputs and keeps the
 * partial-argmax scratch in a fixed 1 MiB device array inside the library (held by every GPU that
 * loads the library, until the process exits).
 *   x [rows][1024] bf16, embed [vocab][1024] bf16, tokens [rows] int32; rows <= 16,
 *   vocab <= 262,144 and a multiple of 8 - larger sizes are refused with Q35_ERR_CAPACITY.
 * The first call on each device looks up the array's device address (with that device current);
 * make that first call before starting any stream capture, and do not let two first calls on the same
 * device run concurrently from two host threads (both would store the same address, but the look-up
 * itself is not meant to be raced).  All calls share the one array: two
 * calls that may overlap on the GPU (different streams, no dependency) race on it.  Calls never
 * allocate or free: no cudaMalloc / cudaFree, and no library routine that allocates. */
int q35_lm_head_argmax_static(const uint16_t* x, const uint16_t* embed, int vocab, int rows,
                              int* tokens, void* stream);
/* gdn_conv + gdn_gates + gdn_rec + gdn_gated_norm (engine/kernels.h:398-460,682) for `lanes`
 * lanes x T tokens of ONE layer.  proj [lanes*T][8224] = [qkv 6144 | z 2048 | b 16 | a 16];
 * S f32 [lanes][16][128][128]; window bf16 [lanes][3][6144]; y [lanes*T][2048].
 * T < 32: token-by-token recurrence (the decode form).  T >= 32: the chunk-64 scan of the
 * reference's prefill (speccheck/specimpl.py:187-235), which overwrites the q|k|v columns of proj
 * with the conv outputs. */
int q35_op_gdn_step(uint16_t* proj, const uint16_t* conv_w, const uint16_t* A_log,
                    const uint16_t* dt_bias, const uint16_t* norm_w, float* S, uint16_t* window,
                    uint16_t* y, int lanes, int T, void* stream);
/* attn_decode_layer (engine/kernels.h:730-906) for `lanes` lanes x T new tokens of ONE layer over a
 * paged cache: proj [lanes*T][5120] = [q|gate per head 4096 | k 512 | v 512]; kpool / vpool are
 * arrays of pages, each bf16 [2 kv heads][64 positions][256]; page_table [lanes][pages_per_lane]
 * page ids; ctx [lanes] = positions already cached (= slot and rope position of the first new
 * token); out [lanes*T][2048] gated attention rows.  Appends the new K/V rows to the cache. */
int q35_op_attn_decode(q35_engine* e, const uint16_t* proj, const uint16_t* q_norm,
                       const uint16_t* k_norm, uint16_t* kpool, uint16_t* vpool,
                       const int* page_table, int pages_per_lane, const int* ctx, uint16_t* out,
                       int lanes, int T, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* Q35_ENGINE_H */
