// tcgen05 / TMEM form of the batched projections for bodies of many rows:
//   out[rows][N] = x[rows][K] . W[N][K]^T   (bf16 operands, f32 accumulate in tensor memory)
//
// One CTA computes a 128-row x BN-column output tile.  Operands arrive by TMA
// (cp.async.bulk.tensor, 128-byte swizzle) into a shared-memory ring (3 stages when two CTAs share
// an SM, 6-8 when the grid is small and latency-bound); one elected thread
// issues tcgen05.mma (M = 128, N = BN, K = 16 per instruction) with the accumulator in tensor
// memory; four epilogue warps read the accumulator back with tcgen05.ld (thread = output row) and
// apply the plain / SwiGLU / argmax epilogue from registers.  Warp roles: 0 = TMA producer,
// 1 = TMEM owner + MMA issuer, 2..5 = epilogue.  With the 3-stage ring two CTAs fit per SM, so one
// tile's epilogue overlaps the other's main loop.  Narrow outputs (N = 1024) at few rows are split
// along K over gridDim.z; each split stores an f32 partial tile and the consumer (the residual
// add + norm kernel) sums the partials in a fixed order.  No cluster multicast is used anywhere.
//
// Every mbarrier wait is bounded (about one second); on expiry the kernel raises the status word,
// skips its stores, still frees its tensor memory and returns.
#include <cuda.h>

#include <cmath>
#include <cstdlib>

#include "q35_common.cuh"
#include "q35_async.cuh"
#include "q35_tcgen05.cuh"

namespace q35 {

namespace {

constexpr int BM = 128, BK = 64;
constexpr int A_BYTES = BM * BK * 2;                 // 16 KiB
constexpr int NUM_THREADS = 192;

// SwiGLU with the reference's three roundings.  SiLU of the bf16-valued gate is rounded to bf16 at
// once, so the fast exponential and divide (a few f32 ULP) change the rounded value in about one
// element in 10^4; the IEEE forms cost this epilogue 3.6 us per 128 x 64 tile (4.9 -> 1.3 us).
__device__ __forceinline__ uint16_t swiglu_bf16(float gate_acc, float up_acc) {
    const float g = bfround(gate_acc);
    const float u = bfround(up_acc);
    const float s = bfround(__fdividef(g, 1.0f + __expf(-g)));
    return f2bf(s * u);
}

// Epilogue of 32 accumulator columns [col0, col0 + 32) of one output row, from registers.
// PARTIAL: f32 partial tile of K split `split`; PLAIN: bf16; SWIGLU: interleaved (gate, up) pairs ->
// bf16 activations; ARGMAX: running (value, lowest index) plus optional f32 logits.
template <int EPI>
__device__ __forceinline__ void epi_chunk(const uint32_t (&r)[32], void* __restrict__ out, float* __restrict__ logits,
                                          int M, int N, int row, int col0, int split, float& bv, int& bi) {
    const int valid = (N - col0) < 32 ? (N - col0) : 32;
    if (EPI == EPI_PARTIAL) {
        float* o = static_cast<float*>(out) + ((size_t)split * M + row) * N + col0;
        if (valid == 32) {
#pragma unroll
            for (int v = 0; v < 8; ++v)
                reinterpret_cast<uint4*>(o)[v] = make_uint4(r[4 * v], r[4 * v + 1], r[4 * v + 2], r[4 * v + 3]);
        } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
                if (j < valid) o[j] = __uint_as_float(r[j]);
        }
    } else if (EPI == EPI_PLAIN) {
        uint16_t* o = static_cast<uint16_t*>(out) + (size_t)row * N + col0;
        if (valid == 32) {
#pragma unroll
            for (int v = 0; v < 4; ++v) {
                uint4 w;
                w.x = pack_bf2(__uint_as_float(r[8 * v + 0]), __uint_as_float(r[8 * v + 1]));
                w.y = pack_bf2(__uint_as_float(r[8 * v + 2]), __uint_as_float(r[8 * v + 3]));
                w.z = pack_bf2(__uint_as_float(r[8 * v + 4]), __uint_as_float(r[8 * v + 5]));
                w.w = pack_bf2(__uint_as_float(r[8 * v + 6]), __uint_as_float(r[8 * v + 7]));
                reinterpret_cast<uint4*>(o)[v] = w;
            }
        } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
                if (j < valid) o[j] = f2bf(__uint_as_float(r[j]));
        }
    } else if (EPI == EPI_SWIGLU) {
        uint16_t* o = static_cast<uint16_t*>(out) + (size_t)row * (N >> 1) + (col0 >> 1);
        if (valid == 32) {
#pragma unroll
            for (int v = 0; v < 2; ++v) {
                uint32_t w[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int b = 16 * v + 4 * j;
                    w[j] = (uint32_t)swiglu_bf16(__uint_as_float(r[b]), __uint_as_float(r[b + 1])) |
                           ((uint32_t)swiglu_bf16(__uint_as_float(r[b + 2]), __uint_as_float(r[b + 3])) << 16);
                }
                reinterpret_cast<uint4*>(o)[v] = make_uint4(w[0], w[1], w[2], w[3]);
            }
        } else {
#pragma unroll
            for (int j = 0; j < 16; ++j)
                if (2 * j + 1 < valid)
                    o[j] = swiglu_bf16(__uint_as_float(r[2 * j]), __uint_as_float(r[2 * j + 1]));
        }
    } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) {
            const float v = __uint_as_float(r[j]);
            if (j < valid && v > bv) { bv = v; bi = col0 + j; }      // ascending scan: lowest id on ties
        }
        if (logits != nullptr) {
            float* lg = logits + (size_t)row * N + col0;
#pragma unroll
            for (int j = 0; j < 32; ++j)
                if (j < valid) lg[j] = __uint_as_float(r[j]);
        }
    }
}

template <int BN, int STAGES, int EPI>
__global__ void __launch_bounds__(NUM_THREADS)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tma_x, const __grid_constant__ CUtensorMap tma_w,
               void* __restrict__ out, int M, int N, int num_kb_total, ArgMax* __restrict__ partials,
               float* __restrict__ logits, int n_parts, int* __restrict__ status, int x_box_bytes) {
    constexpr int B_BYTES = BN * BK * 2;
    constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    // bytes one stage receives: the x box covers only the body's rows when there are fewer than 128 (the rest of
    // the 128-row A tile keeps whatever the shared memory held: those accumulator rows are never stored)
    const uint32_t tx_bytes = (uint32_t)x_box_bytes + B_BYTES;
    constexpr uint32_t IDESC = instr_desc(BM, BN);

    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) unsigned long long bars[2 * STAGES + 1];
    __shared__ uint32_t tmem_base_s;
    __shared__ int abort_s;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid == 0) { prefetch_tensormap(&tma_w); prefetch_tensormap(&tma_x); }
    const int m0 = blockIdx.x * BM, n0 = blockIdx.y * BN;
    // K split: this CTA covers k-blocks [kb0, kb0 + num_kb)
    const int kb_per = (num_kb_total + gridDim.z - 1) / gridDim.z;
    const int kb0 = blockIdx.z * kb_per;
    const int num_kb = (num_kb_total - kb0) < kb_per ? (num_kb_total - kb0) : kb_per;
    const int pre = num_kb < STAGES ? num_kb : STAGES;                 // stages filled before the first wait
    const uint32_t tiles = (smem_u32(smem_raw) + 1023u) & ~1023u;      // 1024-byte aligned ring
    const uint32_t full0 = smem_u32(&bars[0]), empty0 = smem_u32(&bars[STAGES]), accum = smem_u32(&bars[2 * STAGES]);

    if (tid == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
        mbar_init(accum, 1);
        abort_s = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        // weight tiles of the first stages: no kernel writes weights, so these loads may fly while
        // the kernel that produces x is still running
        for (int kb = 0; kb < pre; ++kb) {
            mbar_expect_tx(full0 + 8 * kb, tx_bytes);
            tma_load_2d(tiles + kb * STAGE_BYTES + A_BYTES, &tma_w, (kb0 + kb) * BK, n0, full0 + 8 * kb);
        }
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n"
                     ::"r"(smem_u32(&tmem_base_s)), "r"((uint32_t)BN) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_s;
    // barrier set-up, the tensor-memory allocation and the weight loads above overlap the predecessor's tail
    pdl_wait();
    // an earlier kernel gave up: move no data beyond the loads already in flight, compute nothing
    const bool dead = status != nullptr && *status != 0;

    if (warp == 0) {
        if (lane == 0) {
            for (int kb = 0; kb < pre; ++kb)
                tma_load_2d(tiles + kb * STAGE_BYTES, &tma_x, (kb0 + kb) * BK, m0, full0 + 8 * kb);
            for (int kb = pre; kb < num_kb && !dead; ++kb) {
                const int s = kb % STAGES;
                const uint32_t ph = (kb / STAGES) & 1;
                if (!mbar_wait(empty0 + 8 * s, ph ^ 1)) { abort_s = 1; if (status) atomicExch(status, 2); break; }
                const uint32_t a = tiles + s * STAGE_BYTES;
                mbar_expect_tx(full0 + 8 * s, tx_bytes);
                tma_load_2d(a, &tma_x, (kb0 + kb) * BK, m0, full0 + 8 * s);
                tma_load_2d(a + A_BYTES, &tma_w, (kb0 + kb) * BK, n0, full0 + 8 * s);
            }
            pdl_trigger();               // every load of this CTA is issued: the successor may start
        }
    } else if (warp == 1) {
        if (lane == 0) {
            bool ok = true;
            const int n_wait = dead ? pre : num_kb;      // a dead CTA still lets its own copies land
            for (int kb = 0; kb < n_wait && ok; ++kb) {
                const int s = kb % STAGES;
                const uint32_t ph = (kb / STAGES) & 1;
                if (!mbar_wait(full0 + 8 * s, ph)) { abort_s = 1; if (status) atomicExch(status, 3); ok = false; break; }
                if (dead) continue;
                tc_fence_after();
                const uint32_t a = tiles + s * STAGE_BYTES;
#pragma unroll
                for (int k = 0; k < BK / 16; ++k)
                    tc_mma(tmem_base, smem_desc_sw128(a + k * 32), smem_desc_sw128(a + A_BYTES + k * 32), IDESC,
                           (kb | k) != 0 ? 1u : 0u);
                tc_commit(empty0 + 8 * s);       // frees the stage once these MMAs have read it
            }
            if (ok && !dead) tc_commit(accum);   // accumulator complete
        }
    } else {
        // ---- epilogue: thread = output row (TMEM lane), registers = columns ----------------------
        const bool ready = __all_sync(0xffffffffu, !dead && mbar_wait(accum, 0));
        if (!ready && !dead && lane == 0 && status) atomicExch(status, 4);
        tc_fence_after();
        const int q = warp & 3;                                  // TMEM lane quarter this warp may read
        const int row = m0 + q * 32 + lane;
        float bv = -INFINITY;
        int bi = 0x7fffffff;
        if (ready) {
#pragma unroll 1
            for (int c = 0; c < BN / 32; ++c) {
                uint32_t r[32];
                tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + c * 32, r);
                const int col0 = n0 + c * 32;
                if (row >= M || col0 >= N) continue;
                epi_chunk<EPI>(r, out, logits, M, N, row, col0, blockIdx.z, bv, bi);
            }
            if (EPI == EPI_ARGMAX && row < M) partials[(size_t)row * n_parts + blockIdx.y] = ArgMax{bv, bi};
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"((uint32_t)BN) : "memory");
    }
}

// ------------------------------------------------------------------------------------------------
// Persistent form for bodies with about a wave of tiles or more: one CTA per SM walks 128 x 256 output
// tiles (row tile fastest, so the CTAs that run together share a weight tile through L2).  The
// accumulator is double-buffered in tensor memory (2 x 256 columns): the eight epilogue warps drain
// tile i while the MMA thread fills tile i + 1, and the TMA ring runs on across tile borders, so the
// per-tile ramp (barrier set-up, allocation, first-load latency) is paid once per CTA.
// Warps: 0 = TMA producer, 1 = TMEM owner + MMA issuer, 2..9 = epilogue (lane quarter = warp % 4,
// column half = (warp - 2) / 4).  Any wait that runs out raises the status word and an abort flag
// that every other wait polls; the CTA then lets its copies in flight land, frees its tensor
// memory and returns.
// ------------------------------------------------------------------------------------------------
constexpr int P_THREADS = 320;
constexpr int P_BN = 256;

__device__ __forceinline__ bool mbar_wait_or_abort(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
    unsigned long long t0 = 0;
    for (int it = 0;; ++it) {
        uint32_t ok;
        asm volatile(
            "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
            " selp.u32 %0, 1, 0, p;\n}\n"
            : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
        if (ok) return true;
        if (*abort_flag) return false;
        if (it == 0) t0 = global_ns();
        else if (global_ns() - t0 > 1000000000ull) return false;
    }
}
template <int STAGES, int EPI>
__global__ void __launch_bounds__(P_THREADS, 1)
gemm_tc_persist_kernel(const __grid_constant__ CUtensorMap tma_x, const __grid_constant__ CUtensorMap tma_w,
                       void* __restrict__ out, int M, int N, int num_kb, int m_tiles, int n_tiles,
                       ArgMax* __restrict__ partials, float* __restrict__ logits, int n_parts,
                       int* __restrict__ status) {
    constexpr int B_BYTES = P_BN * BK * 2;
    constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    constexpr uint32_t IDESC = instr_desc(BM, P_BN);

    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) unsigned long long bars[2 * STAGES + 5];
    __shared__ uint32_t tmem_base_s;
    __shared__ volatile int abort_s;
    __shared__ int issued_s, consumed_s;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid == 0) { prefetch_tensormap(&tma_w); prefetch_tensormap(&tma_x); }
    const int total = m_tiles * n_tiles;
    const uint32_t tiles = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t full0 = smem_u32(&bars[0]), empty0 = smem_u32(&bars[STAGES]);
    const uint32_t accf0 = smem_u32(&bars[2 * STAGES]), acce0 = smem_u32(&bars[2 * STAGES + 2]);
    const uint32_t drain = smem_u32(&bars[2 * STAGES + 4]);
    const int first = blockIdx.x;
    const int pre = (first < total) ? (num_kb < STAGES ? num_kb : STAGES) : 0;

    if (tid == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
        mbar_init(accf0, 1); mbar_init(accf0 + 8, 1);
        mbar_init(acce0, 8); mbar_init(acce0 + 8, 8);
        mbar_init(drain, 1);
        abort_s = 0; issued_s = 0; consumed_s = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        // weight tiles of the first stages fly while the kernel that produces x is still running
        const int n0 = (first / m_tiles) * P_BN;
        for (int kb = 0; kb < pre; ++kb) {
            mbar_expect_tx(full0 + 8 * kb, STAGE_BYTES);
            tma_load_2d(tiles + kb * STAGE_BYTES + A_BYTES, &tma_w, kb * BK, n0, full0 + 8 * kb);
        }
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n"
                     ::"r"(smem_u32(&tmem_base_s)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_s;
    pdl_wait();
    const bool dead = status != nullptr && *status != 0;      // an earlier kernel gave up
    const int my_last = dead ? (pre > 0 ? first + 1 : first) : total;   // a dead CTA only lets its copies land

    if (warp == 0) {
        if (lane == 0) {
            int it = 0;
            bool ok = true;
            for (int tile = first; tile < my_last && ok; tile += gridDim.x) {
                const int m0 = (tile % m_tiles) * BM, n0 = (tile / m_tiles) * P_BN;
                const int kb_end = dead ? pre : num_kb;
                for (int kb = 0; kb < kb_end; ++kb, ++it) {
                    const int s = it % STAGES;
                    const uint32_t a = tiles + s * STAGE_BYTES;
                    if (it < pre) {                       // weights already under way: add the rows of x
                        tma_load_2d(a, &tma_x, kb * BK, m0, full0 + 8 * s);
                        continue;
                    }
                    if (!mbar_wait_or_abort(empty0 + 8 * s, ((it / STAGES) & 1) ^ 1, &abort_s)) {
                        abort_s = 1; if (status) atomicExch(status, 2); ok = false; break;
                    }
                    mbar_expect_tx(full0 + 8 * s, STAGE_BYTES);
                    tma_load_2d(a, &tma_x, kb * BK, m0, full0 + 8 * s);
                    tma_load_2d(a + A_BYTES, &tma_w, kb * BK, n0, full0 + 8 * s);
                }
            }
            issued_s = it;
            pdl_trigger();               // every load of this CTA is issued: the successor may start
        }
    } else if (warp == 1) {
        if (lane == 0) {
            int it = 0, i = 0;
            bool ok = true;
            for (int tile = first; tile < my_last && ok; tile += gridDim.x, ++i) {
                const int buf = i & 1;
                const uint32_t d_tmem = tmem_base + buf * P_BN;
                if (!dead && !mbar_wait_or_abort(acce0 + 8 * buf, ((i >> 1) & 1) ^ 1, &abort_s)) {
                    abort_s = 1; if (status) atomicExch(status, 5); ok = false; break;
                }
                tc_fence_after();
                const int kb_end = dead ? pre : num_kb;
                for (int kb = 0; kb < kb_end; ++kb, ++it) {
                    const int s = it % STAGES;
                    if (!mbar_wait_or_abort(full0 + 8 * s, (it / STAGES) & 1, &abort_s)) {
                        abort_s = 1; if (status) atomicExch(status, 3); ok = false; break;
                    }
                    if (dead) continue;
                    tc_fence_after();
                    const uint32_t a = tiles + s * STAGE_BYTES;
#pragma unroll
                    for (int k = 0; k < BK / 16; ++k)
                        tc_mma(d_tmem, smem_desc_sw128(a + k * 32), smem_desc_sw128(a + A_BYTES + k * 32), IDESC,
                               (kb | k) != 0 ? 1u : 0u);
                    tc_commit(empty0 + 8 * s);           // frees the stage once these MMAs have read it
                }
                if (ok && !dead) tc_commit(accf0 + 8 * buf);
            }
            consumed_s = it;
            if (!ok) {                                   // let the MMAs already issued finish before the memory goes
                tc_commit(drain);
                mbar_wait(drain, 0);
            }
        }
    } else if (!dead) {
        // ---- epilogue: thread = output row (TMEM lane), 32-column chunks of this warp's column half ----
        const int q = warp & 3, ch = (warp - 2) >> 2;
        int i = 0;
        for (int tile = first; tile < total; tile += gridDim.x, ++i) {
            const int buf = i & 1;
            const int m0 = (tile % m_tiles) * BM, n0 = (tile / m_tiles) * P_BN + ch * (P_BN / 2);
            // one outcome for the whole warp: tcgen05.ld below needs all 32 lanes
            if (!__all_sync(0xffffffffu, mbar_wait_or_abort(accf0 + 8 * buf, (i >> 1) & 1, &abort_s))) {
                if (lane == 0) { abort_s = 1; if (status) atomicExch(status, 4); }
                break;
            }
            tc_fence_after();
            const int row = m0 + q * 32 + lane;
            float bv = -INFINITY;
            int bi = 0x7fffffff;
#pragma unroll 1
            for (int c = 0; c < P_BN / 64; ++c) {
                uint32_t r[32];
                tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + buf * P_BN + ch * (P_BN / 2) + c * 32, r);
                const int col0 = n0 + c * 32;
                if (row >= M || col0 >= N) continue;
                epi_chunk<EPI>(r, out, logits, M, N, row, col0, 0, bv, bi);
            }
            // this warp has read its part of the accumulator: hand the buffer back to the MMA thread
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(acce0 + 8 * buf);
            if (EPI == EPI_ARGMAX && row < M && n0 < N) partials[(size_t)row * n_parts + (n0 >> 7)] = ArgMax{bv, bi};
        }
    }

    tc_fence_before();
    __syncthreads();
    if (tid == 0 && abort_s) {
        // copies issued but never consumed must land before the shared memory is given up
        for (int k = consumed_s; k < issued_s; ++k) mbar_wait(full0 + 8 * (k % STAGES), (k / STAGES) & 1);
    }
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(512u) : "memory");
    }
}

// ---- the tied head for bodies of at most 32 rows: the TABLE is the M operand --------------------------
// logits^T [vocab][rows] = table [vocab][K] . x [rows][K]^T : A = 128 table rows of one k-block (K-major, by TMA),
// B = the body's rows (N = NB = 16 or 32 columns of the MMA; rows past the body are zero-filled by TMA, once),
// D = 128 lanes x NB columns of tensor memory, double-buffered.  The x rows for ALL of K (16 k-blocks x NB x 128 B) are
// loaded once per CTA and stay, so a ring stage holds nothing but 16 KiB of the table and eleven (NB = 16) or nine
// of them are in flight per SM (with 64 columns only five fit and the per-row reduction shows: 152 us; not built); the
// form with x as the M operand moved a 16 KiB x tile of which at most one eighth was real through every stage and
// did sixteen times the tensor-pipe work (116 -> 82 us per 1-row head = 6.2 TB/s).  Warp roles: 0 = TMA producer, 1 = tensor
// memory owner + MMA issuer, 2..5 = epilogue: thread = one table row of the tile, its NB accumulator columns are the
// logits of that token id for the body's rows; optional f32 logits stores (coalesced along the vocabulary), then per
// body row a (value, lowest id) reduction over the warp's 32 ids by shuffles and over the four warps through shared
// memory: one partial per (row, 128-id tile), as the other head forms write.
constexpr int H_THREADS = 192, H_KB = 16, H_MAX_NB = 32;
__host__ __device__ constexpr int head_stages(int nb) { return nb <= 16 ? 11 : 9; }
constexpr size_t head_smem(int nb) { return (size_t)head_stages(nb) * A_BYTES + (size_t)H_KB * nb * 128 + 1024; }

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
}

template <int H_NB>
__global__ void __launch_bounds__(H_THREADS, 1)
head_rows_tc_kernel(const __grid_constant__ CUtensorMap tma_x, const __grid_constant__ CUtensorMap tma_w, int M, int N,
                    int n_tiles, ArgMax* __restrict__ partials, float* __restrict__ logits, int n_parts,
                    int* __restrict__ status) {
    static_assert(H_NB == 16 || H_NB == 32, "one body row per lane of an epilogue warp");
    constexpr uint32_t IDESC = instr_desc(BM, H_NB);
    constexpr int H_STAGES = head_stages(H_NB);
    constexpr int H_XBYTES = H_KB * H_NB * 128;              // [k-block][NB rows][128 B]
    constexpr uint32_t TMEM_COLS = 2 * H_NB < 32 ? 32 : 2 * H_NB;
    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) unsigned long long bars[2 * H_STAGES + 6];
    __shared__ uint32_t tmem_base_s;
    __shared__ volatile int abort_s;
    __shared__ int issued_s, consumed_s, x_issued_s, x_waited_s;
    __shared__ float wb_v[2][4][H_NB];
    __shared__ int wb_i[2][4][H_NB];

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid == 0) { prefetch_tensormap(&tma_w); prefetch_tensormap(&tma_x); }
    const uint32_t ring = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t xs = ring + H_STAGES * A_BYTES;
    const uint32_t full0 = smem_u32(&bars[0]), empty0 = smem_u32(&bars[H_STAGES]);
    const uint32_t accf0 = smem_u32(&bars[2 * H_STAGES]), acce0 = smem_u32(&bars[2 * H_STAGES + 2]);
    const uint32_t xfull = smem_u32(&bars[2 * H_STAGES + 4]), drain = smem_u32(&bars[2 * H_STAGES + 5]);
    const int first = blockIdx.x;
    const int pre = first < n_tiles ? (H_KB < H_STAGES ? H_KB : H_STAGES) : 0;

    if (tid == 0) {
        for (int s = 0; s < H_STAGES; ++s) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
        mbar_init(accf0, 1); mbar_init(accf0 + 8, 1);
        mbar_init(acce0, 4); mbar_init(acce0 + 8, 4);
        mbar_init(xfull, 1); mbar_init(drain, 1);
        abort_s = 0; issued_s = 0; consumed_s = 0; x_issued_s = 0; x_waited_s = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        // table tiles of the first stages fly while the kernel that produces x is still running
        for (int kb = 0; kb < pre; ++kb) {
            mbar_expect_tx(full0 + 8 * kb, A_BYTES);
            tma_load_2d(ring + kb * A_BYTES, &tma_w, kb * BK, first * BM, full0 + 8 * kb);
        }
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n"
                     ::"r"(smem_u32(&tmem_base_s)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_s;
    pdl_wait();
    const bool dead = status != nullptr && *status != 0;      // an earlier kernel gave up
    const int my_last = dead ? (pre > 0 ? first + 1 : first) : n_tiles;   // a dead CTA only lets its copies land

    if (warp == 0) {
        if (lane == 0) {
            if (!dead && first < n_tiles) {
                mbar_expect_tx(xfull, H_XBYTES);
                for (int kb = 0; kb < H_KB; ++kb) tma_load_2d(xs + kb * (H_NB * 128), &tma_x, kb * BK, 0, xfull);
                x_issued_s = 1;
            }
            int it = 0;
            bool ok = true;
            for (int tile = first; tile < my_last && ok; tile += gridDim.x) {
                const int kb_end = dead ? pre : H_KB;
                for (int kb = 0; kb < kb_end; ++kb, ++it) {
                    if (it < pre) continue;                   // issued ahead of the wait
                    const int s = it % H_STAGES;
                    if (!mbar_wait_or_abort(empty0 + 8 * s, ((it / H_STAGES) & 1) ^ 1, &abort_s)) {
                        abort_s = 1; if (status) atomicExch(status, 2); ok = false; break;
                    }
                    mbar_expect_tx(full0 + 8 * s, A_BYTES);
                    tma_load_2d(ring + s * A_BYTES, &tma_w, kb * BK, tile * BM, full0 + 8 * s);
                }
            }
            issued_s = it;
            pdl_trigger();               // every load of this CTA is issued: the successor may start
        }
    } else if (warp == 1) {
        if (lane == 0) {
            int it = 0, i = 0;
            bool ok = true;
            if (!dead && first < n_tiles) {
                if (!mbar_wait_or_abort(xfull, 0, &abort_s)) { abort_s = 1; if (status) atomicExch(status, 3); ok = false; }
                else x_waited_s = 1;
            }
            for (int tile = first; tile < my_last && ok; tile += gridDim.x, ++i) {
                const int buf = i & 1;
                const uint32_t d_tmem = tmem_base + buf * H_NB;
                if (!dead && !mbar_wait_or_abort(acce0 + 8 * buf, ((i >> 1) & 1) ^ 1, &abort_s)) {
                    abort_s = 1; if (status) atomicExch(status, 5); ok = false; break;
                }
                tc_fence_after();
                const int kb_end = dead ? pre : H_KB;
                for (int kb = 0; kb < kb_end; ++kb, ++it) {
                    const int s = it % H_STAGES;
                    if (!mbar_wait_or_abort(full0 + 8 * s, (it / H_STAGES) & 1, &abort_s)) {
                        abort_s = 1; if (status) atomicExch(status, 3); ok = false; break;
                    }
                    if (dead) continue;
                    tc_fence_after();
                    const uint32_t a = ring + s * A_BYTES, b = xs + kb * (H_NB * 128);
#pragma unroll
                    for (int k = 0; k < BK / 16; ++k)
                        tc_mma(d_tmem, smem_desc_sw128(a + k * 32), smem_desc_sw128(b + k * 32), IDESC, (kb | k) != 0 ? 1u : 0u);
                    tc_commit(empty0 + 8 * s);           // frees the stage once these MMAs have read it
                }
                if (ok && !dead) tc_commit(accf0 + 8 * buf);
            }
            consumed_s = it;
            if (!ok) {                                   // let the MMAs already issued finish before the memory goes
                tc_commit(drain);
                mbar_wait(drain, 0);
            }
        }
    } else if (!dead) {
        // ---- epilogue: thread = table row (tensor-memory lane) of the tile ----
        const int q = warp & 3, ew = warp - 2;
        int i = 0;
        bool live = true;
        for (int tile = first; tile < n_tiles; tile += gridDim.x, ++i) {
            const int buf = i & 1;
            // one outcome for the whole warp: tcgen05.ld below needs all 32 lanes
            if (live && !__all_sync(0xffffffffu, mbar_wait_or_abort(accf0 + 8 * buf, (i >> 1) & 1, &abort_s))) {
                if (lane == 0) { abort_s = 1; if (status) atomicExch(status, 4); }
                live = false;
            }
            float myv = -INFINITY;
            int myi = 0x7fffffff;
            if (live) {
                tc_fence_after();
                const int n = tile * BM + q * 32 + lane;
                const bool n_ok = n < N;
#pragma unroll
                for (int c = 0; c < H_NB / 16; ++c) {
                    uint32_t r[16];
                    tmem_ld16(tmem_base + ((uint32_t)(q * 32) << 16) + buf * H_NB + c * 16, r);
                    if (c == H_NB / 16 - 1) {
                        // this warp has read its part of the accumulator: hand the buffer back to the MMA thread
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(acce0 + 8 * buf);
                    }
#pragma unroll
                    for (int jj = 0; jj < 16; ++jj) {
                        const int j = c * 16 + jj;
                        if (j >= M) break;                 // M is the same for every thread
                        const float v = __uint_as_float(r[jj]);
                        if (logits != nullptr && n_ok) logits[(size_t)j * N + n] = v;
                        float bv = n_ok ? v : -INFINITY;
                        int bi = n_ok ? n : 0x7fffffff;
#pragma unroll
                        for (int o = 16; o > 0; o >>= 1) {
                            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
                            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
                            if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
                        }
                        if (lane == j) { myv = bv; myi = bi; }      // lane j keeps the winner of body row j
                    }
                }
            }
            // the four warps' winners meet in shared memory (all four run this barrier for every tile of the CTA)
            if (lane < H_NB) { wb_v[buf][ew][lane] = myv; wb_i[buf][ew][lane] = myi; }
            asm volatile("bar.sync 1, 128;\n" ::: "memory");
            const int et = ew * 32 + lane;                 // epilogue thread: one body row each
            if (et < M && !abort_s) {
                float bv = wb_v[buf][0][et];
                int bi = wb_i[buf][0][et];
#pragma unroll
                for (int w = 1; w < 4; ++w) {
                    const float ov = wb_v[buf][w][et];
                    const int oi = wb_i[buf][w][et];
                    if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
                }
                partials[(size_t)et * n_parts + tile] = ArgMax{bv, bi};
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (tid == 0 && abort_s) {
        // copies issued but never consumed must land before the shared memory is given up
        for (int k = consumed_s; k < issued_s; ++k) mbar_wait(full0 + 8 * (k % H_STAGES), (k / H_STAGES) & 1);
        if (x_issued_s && !x_waited_s) mbar_wait(xfull, 0);
    }
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

// ---- projections of bodies of 17 - 32 rows with K = 1024: the WEIGHTS are the M operand -------------------------
// out^T [N][rows]: a CTA owns 64 weight rows and holds ALL of their K in shared memory (16 k-blocks x 8 KiB), fetched
// by TMA before the programmatic-launch wait - weights are immutable, so the whole tile flies while the kernel that
// produces x still runs, as in the weight-streaming kernel of <= 16 rows.  After the wait only the body's rows (B
// operand, N = 32 columns of the MMA, 16 boxes of 4 KiB) have to arrive; the MMAs follow them k-group by k-group.
// tcgen05.mma runs with M = 128 on the 64-row tile (the upper 64 accumulator lanes see whatever lies behind the tile
// in shared memory and are never read), so the accumulator layout is lane = weight row.  Epilogue warps with lanes
// 0 - 63 turn their 32 columns into bf16, transpose through shared memory and store rows of the output with 16-byte
// stores.  Every wait is bounded.  In-projection piece 6144 x 1024 at 32 rows: 5.4 us against 7.2 us for the form with
// x as the M operand (launches replayed back to back); inside a step the two forms tie.
constexpr int R_THREADS = 192, R_NB = 32, R_KB = 16, R_BM = 64, R_GROUPS = 4;
constexpr int R_WBYTES = R_KB * R_BM * 128, R_XBYTES = R_KB * R_NB * 128;          // 128 KiB + 64 KiB
constexpr size_t kRowsSmem = (size_t)R_WBYTES + R_XBYTES + 1024;      // the M = 128 read of the last k-block overhangs into x

template <int EPI>
__global__ void __launch_bounds__(R_THREADS, 1)
proj_rows_tc_kernel(const __grid_constant__ CUtensorMap tma_x, const __grid_constant__ CUtensorMap tma_w,
                    uint16_t* __restrict__ out, int M, int N, int* __restrict__ status) {
    constexpr uint32_t IDESC = instr_desc(128, R_NB);
    static_assert(EPI == EPI_PLAIN, "bf16 store epilogue only");
    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) unsigned long long bars[2 * R_GROUPS + 1];
    __shared__ uint32_t tmem_base_s;
    __shared__ int x_issued_s;
    __shared__ volatile int abort_s;
    __shared__ __align__(16) uint16_t tile_s[R_NB][R_BM + 8];                      // [body row][output column]

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid == 0) { prefetch_tensormap(&tma_w); prefetch_tensormap(&tma_x); }
    const uint32_t ws = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t xs = ws + R_WBYTES;
    const uint32_t wfull0 = smem_u32(&bars[0]), xfull0 = smem_u32(&bars[R_GROUPS]), accum = smem_u32(&bars[2 * R_GROUPS]);
    const int n0 = blockIdx.x * R_BM;
    constexpr int KB_PER = R_KB / R_GROUPS;

    if (tid == 0) {
        for (int g = 0; g < R_GROUPS; ++g) { mbar_init(wfull0 + 8 * g, 1); mbar_init(xfull0 + 8 * g, 1); }
        mbar_init(accum, 1);
        x_issued_s = 0; abort_s = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        for (int g = 0; g < R_GROUPS; ++g) {
            mbar_expect_tx(wfull0 + 8 * g, KB_PER * R_BM * 128);
            for (int kb = g * KB_PER; kb < (g + 1) * KB_PER; ++kb)
                tma_load_2d(ws + kb * (R_BM * 128), &tma_w, kb * BK, n0, wfull0 + 8 * g);
        }
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n"
                     ::"r"(smem_u32(&tmem_base_s)), "r"((uint32_t)R_NB) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_s;
    pdl_wait();
    const bool dead = status != nullptr && *status != 0;      // an earlier kernel gave up: only let the copies land

    if (warp == 0) {
        if (lane == 0) {
            if (!dead) {
                for (int g = 0; g < R_GROUPS; ++g) {
                    mbar_expect_tx(xfull0 + 8 * g, KB_PER * R_NB * 128);
                    for (int kb = g * KB_PER; kb < (g + 1) * KB_PER; ++kb)
                        tma_load_2d(xs + kb * (R_NB * 128), &tma_x, kb * BK, 0, xfull0 + 8 * g);
                }
                x_issued_s = 1;
            }
            pdl_trigger();               // every load of this CTA is issued: the successor may start
        }
    } else if (warp == 1) {
        if (lane == 0) {
            for (int g = 0; g < R_GROUPS; ++g) {
                if (!mbar_wait(wfull0 + 8 * g, 0)) { abort_s = 1; if (status) atomicExch(status, 3); break; }
                if (dead) continue;
                if (!mbar_wait(xfull0 + 8 * g, 0)) { abort_s = 1; if (status) atomicExch(status, 3); break; }
                tc_fence_after();
                for (int kb = g * KB_PER; kb < (g + 1) * KB_PER; ++kb) {
                    const uint32_t a = ws + kb * (R_BM * 128), b = xs + kb * (R_NB * 128);
#pragma unroll
                    for (int k = 0; k < BK / 16; ++k)
                        tc_mma(tmem_base, smem_desc_sw128(a + k * 32), smem_desc_sw128(b + k * 32), IDESC, (kb | k) != 0 ? 1u : 0u);
                }
            }
            // arrives when every MMA issued so far has finished (also after a wait that ran out: nothing may still
            // be reading the shared memory when the CTA leaves)
            tc_commit(accum);
        }
    }
    if (warp >= 2) {
        // ---- epilogue: warps 4 and 5 own accumulator lanes 0 - 63 (lane quarter = warp % 4); all four wait ----
        const bool ready = __all_sync(0xffffffffu, mbar_wait(accum, 0));
        if (!ready && lane == 0) { abort_s = 1; if (status) atomicExch(status, 4); }
        tc_fence_after();
        const int q = warp & 3;
        const bool store = ready && !dead && !abort_s;
        if (q < 2 && store) {
            uint32_t r[32];
            tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16), r);
            const int c = q * 32 + lane;                       // weight row of the tile = output column
#pragma unroll
            for (int j = 0; j < R_NB; ++j) tile_s[j][c] = f2bf(__uint_as_float(r[j]));
        }
        asm volatile("bar.sync 1, 128;\n" ::: "memory");
        if (store) {
            // rows of the output: OUT_COLS bf16 per body row, 16-byte stores
            const int et = (warp - 2) * 32 + lane;
            const int ldo = N, o0 = n0;
            constexpr int CH = R_BM / 8;                       // 16-byte chunks per row
            for (int idx = et; idx < M * CH; idx += 128) {
                const int j = idx / CH, ch = idx % CH;
                if (o0 + ch * 8 + 8 <= ldo)
                    *reinterpret_cast<uint4*>(out + (size_t)j * ldo + o0 + ch * 8) = *reinterpret_cast<const uint4*>(&tile_s[j][ch * 8]);
                else
                    for (int e = 0; e < 8; ++e)
                        if (o0 + ch * 8 + e < ldo) out[(size_t)j * ldo + o0 + ch * 8 + e] = tile_s[j][ch * 8 + e];
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (tid == 0 && abort_s) {
        // copies that nobody waited for must land before the shared memory is given up
        for (int g = 0; g < R_GROUPS; ++g) {
            mbar_wait(wfull0 + 8 * g, 0);
            if (x_issued_s) mbar_wait(xfull0 + 8 * g, 0);
        }
    }
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"((uint32_t)R_NB) : "memory");
    }
}

// ---- host side: tensor maps -------------------------------------------------------------------
// bf16 matrix [rows][K] row-major, box = 64 k-elements x box_rows rows, 128-byte swizzle, zero fill
bool make_map(CUtensorMap* map, const void* base, int rows, int K, int box_rows) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (fn == nullptr) return false;
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)K * 2};
    cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
    cuuint32_t elem[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int BN, int STAGES, int EPI>
cudaError_t run_tc(const uint16_t* x, const uint16_t* W, void* out, int M, int N, int K, int splits,
                   ArgMax* partials, float* logits, int n_parts, int* status, cudaStream_t st) {
    constexpr size_t smem = (size_t)STAGES * (A_BYTES + BN * BK * 2) + 1024;
    static bool attr_done[kMaxDevices] = {false};       // per instantiation and device
    auto kern = gemm_tc_kernel<BN, STAGES, EPI>;
    cudaError_t e = opt_in_smem(kern, smem, attr_done);
    if (e != cudaSuccess) return e;
    CUtensorMap mx, mw;
    // a body of fewer than 128 rows: the x box stops at the body's last row (rounded up to 8), so TMA neither
    // fetches nor zero-fills rows that do not exist (a 128-row box of which a quarter was real cost a 32-row
    // projection more than a full 128-row one)
    const int box_rows = M >= BM ? BM : ((M + 7) & ~7);
    if (!make_map(&mx, x, M, K, box_rows) || !make_map(&mw, W, N, K, BN)) return cudaErrorInvalidValue;
    dim3 grid((M + BM - 1) / BM, (N + BN - 1) / BN, splits);
    return launch_k(kern, grid, dim3(NUM_THREADS), smem, st, mx, mw, out, M, N, K / BK, partials, logits, n_parts, status,
                    box_rows * BK * 2);
}

template <int STAGES, int EPI>
cudaError_t run_tc_persist(const uint16_t* x, const uint16_t* W, void* out, int M, int N, int K, int sms,
                           ArgMax* partials, float* logits, int n_parts, int* status, cudaStream_t st) {
    constexpr size_t smem = (size_t)STAGES * (A_BYTES + P_BN * BK * 2) + 1024;
    static bool attr_done[kMaxDevices] = {false};       // per instantiation and device
    auto kern = gemm_tc_persist_kernel<STAGES, EPI>;
    cudaError_t e = opt_in_smem(kern, smem, attr_done);
    if (e != cudaSuccess) return e;
    CUtensorMap mx, mw;
    if (!make_map(&mx, x, M, K, BM) || !make_map(&mw, W, N, K, P_BN)) return cudaErrorInvalidValue;
    const int m_tiles = (M + BM - 1) / BM, n_tiles = (N + P_BN - 1) / P_BN;
    const int total = m_tiles * n_tiles;
    return launch_k(kern, dim3(total < sms ? total : sms), dim3(P_THREADS), smem, st, mx, mw, out, M, N, K / BK,
                    m_tiles, n_tiles, partials, logits, n_parts, status);
}

// the head of at most 32 rows with the table as the M operand (Q35_HEAD_SWAP=0 keeps x as the M operand)
bool head_rows_form(int rows, int N, int K, int epi) {
    static int mode = -1;
    if (mode < 0) {
        const char* env = std::getenv("Q35_HEAD_SWAP");
        mode = (env != nullptr && env[0] == '0') ? 0 : 1;
    }
    return mode == 1 && epi == EPI_ARGMAX && rows <= H_MAX_NB && K == H_KB * BK && N >= BM;
}
template <int NB>
cudaError_t run_head_rows_tc(const uint16_t* x, const uint16_t* W, int M, int N, int K, int sms, ArgMax* partials,
                             float* logits, int n_parts, int* status, cudaStream_t st) {
    static bool attr_done[kMaxDevices] = {false};
    cudaError_t e = opt_in_smem(head_rows_tc_kernel<NB>, head_smem(NB), attr_done);
    if (e != cudaSuccess) return e;
    CUtensorMap mx, mw;
    if (!make_map(&mx, x, M, K, NB) || !make_map(&mw, W, N, K, BM)) return cudaErrorInvalidValue;
    const int n_tiles = (N + BM - 1) / BM;
    if (n_parts < n_tiles) return cudaErrorInvalidValue;
    return launch_k(head_rows_tc_kernel<NB>, dim3(n_tiles < sms ? n_tiles : sms), dim3(H_THREADS), head_smem(NB), st, mx, mw,
                    M, N, n_tiles, partials, logits, n_parts, status);
}

// projections of 17 - 32 rows with K = 1024: the form with the weights as the M operand (Q35_ROWS_SWAP=0: off)
bool proj_rows_form(int rows, int N, int K, int epi) {
    static int mode = -1;
    if (mode < 0) {
        const char* env = std::getenv("Q35_ROWS_SWAP");
        mode = (env != nullptr && env[0] == '0') ? 0 : 1;
    }
    // the gate/up projection stays on the form with x as the M operand: measured 8.7 against 8.4 us at 32 rows
    return mode == 1 && epi == EPI_PLAIN && rows > 16 && rows <= R_NB && K == R_KB * BK && N >= R_BM && (N & 15) == 0;
}
template <int EPI>
cudaError_t run_proj_rows_tc(const uint16_t* x, const uint16_t* W, void* out, int M, int N, int K, int* status, cudaStream_t st) {
    static bool attr_done[kMaxDevices] = {false};
    cudaError_t e = opt_in_smem(proj_rows_tc_kernel<EPI>, kRowsSmem, attr_done);
    if (e != cudaSuccess) return e;
    CUtensorMap mx, mw;
    if (!make_map(&mx, x, M, K, R_NB) || !make_map(&mw, W, N, K, R_BM)) return cudaErrorInvalidValue;
    return launch_k(proj_rows_tc_kernel<EPI>, dim3((N + R_BM - 1) / R_BM), dim3(R_THREADS), kRowsSmem, st, mx, mw,
                    static_cast<uint16_t*>(out), M, N, status);
}

// the persistent form pays from about one wave of 128 x 256 tiles (Q35_GEMM_PERSIST_MIN overrides)
bool use_persist(int rows, int N) {
    static int mode = -1;                                // Q35_GEMM_PERSIST=0 keeps the one-tile-per-CTA form
    if (mode < 0) {
        const char* env = std::getenv("Q35_GEMM_PERSIST");
        mode = (env != nullptr && env[0] == '0') ? 0 : 1;
    }
    if (!mode) return false;
    const int total = ((rows + BM - 1) / BM) * ((N + P_BN - 1) / P_BN);
    static int min_tiles = 0;
    if (min_tiles == 0) {
        const char* env = std::getenv("Q35_GEMM_PERSIST_MIN");
        min_tiles = env != nullptr ? std::atoi(env) : 0;
        if (min_tiles <= 0) min_tiles = 128;             // measured: wins from about one wave of tiles up
    }
    return total >= min_tiles;
}

}  // namespace

bool linear_tc_eligible(int rows, int N, int K) { return rows > 16 && N >= 128 && K % BK == 0; }   // fewer rows than a tile: the x box stops at the body's last row

// K splits the tcgen05 form would use for a plain projection (1 = no split).
int linear_tc_splits(int rows, int N, int K, int max_rows_ws) {
    if (!linear_tc_eligible(rows, N, K) || N > 1024 || rows > max_rows_ws) return 1;
    const int tiles = ((rows + BM - 1) / BM) * ((N + 127) / 128);
    if (tiles >= 100) return 1;
    const int num_kb = K / BK;
    int splits = (sm_count() + tiles - 1) / tiles;
    if (splits > num_kb / 4) splits = num_kb / 4;        // at least 4 k-blocks per split
    if (splits > kMaxSplits) splits = kMaxSplits;
    // Every split writes and the add + norm kernel reads a rows x N f32 partial: the best split count
    // falls with the row count (measured: 8 at 128 rows, 6 at 256, 4 at 512), about 90 / sqrt(rows).
    const int by_rows = (int)lroundf(90.5f / sqrtf((float)rows));
    if (splits > by_rows) splits = by_rows;
    if (splits < 2) return 1;
    const int kb_per = (num_kb + splits - 1) / splits;
    return (num_kb + kb_per - 1) / kb_per;               // every split gets at least one k-block
}

cudaError_t launch_linear_tc_split(const uint16_t* x, const uint16_t* W, float* ws, int rows, int N, int K,
                                   int splits, int* status, cudaStream_t st) {
    return run_tc<128, 4, EPI_PARTIAL>(x, W, ws, rows, N, K, splits, nullptr, nullptr, 0, status, st);
}

// name of the tcgen05 form launch_linear_tc takes (for the benchmark's per-shape report)
const char* linear_tc_route(int rows, int N, int epi) {
    if (proj_rows_form(rows, N, R_KB * BK, epi)) return "proj_rows_tc_kernel (weight rows as the M operand, tile fetched ahead of the wait)";
    if (head_rows_form(rows, N, H_KB * BK, epi)) return rows <= 16 ? "head_rows_tc_kernel<16> (table rows as the M operand, persistent)" : "head_rows_tc_kernel<32> (table rows as the M operand, persistent)";
    const int tiles = ((rows + BM - 1) / BM) * ((N + 127) / 128);
    if (use_persist(rows, N)) return "gemm_tc_persist_kernel (128x256 tiles, persistent)";
    if (epi == EPI_ARGMAX) return "gemm_tc_kernel<128,3>";
    if (tiles < 100) return "gemm_tc_kernel<64,8>";
    if (tiles <= sm_count()) return "gemm_tc_kernel<128,6>";
    return "gemm_tc_kernel<128,3>";
}

cudaError_t launch_linear_tc(const uint16_t* x, const uint16_t* W, void* out, int rows, int N, int K, int epi,
                             ArgMax* partials, float* logits, int n_parts, int* status, cudaStream_t st) {
    if (head_rows_form(rows, N, K, epi)) {
        if (rows <= 16) return run_head_rows_tc<16>(x, W, rows, N, K, sm_count(), partials, logits, n_parts, status, st);
        return run_head_rows_tc<32>(x, W, rows, N, K, sm_count(), partials, logits, n_parts, status, st);
    }
    if (proj_rows_form(rows, N, K, epi)) {
        return run_proj_rows_tc<EPI_PLAIN>(x, W, out, rows, N, K, status, st);
    }
    const int tiles = ((rows + BM - 1) / BM) * ((N + 127) / 128);
    if (use_persist(rows, N)) {
        const int sms = sm_count();
        if (epi == EPI_ARGMAX) return run_tc_persist<4, EPI_ARGMAX>(x, W, out, rows, N, K, sms, partials, logits, n_parts, status, st);
        if (epi == EPI_PLAIN) return run_tc_persist<4, EPI_PLAIN>(x, W, out, rows, N, K, sms, partials, logits, n_parts, status, st);
        if (epi == EPI_SWIGLU) return run_tc_persist<4, EPI_SWIGLU>(x, W, out, rows, N, K, sms, partials, logits, n_parts, status, st);
    }
    if (epi == EPI_ARGMAX)
        return run_tc<128, 3, EPI_ARGMAX>(x, W, out, rows, N, K, 1, partials, logits, n_parts, status, st);
    if (epi == EPI_PLAIN) {
        if (tiles < 100) return run_tc<64, 8, EPI_PLAIN>(x, W, out, rows, N, K, 1, partials, logits, n_parts, status, st);
        if (tiles <= sm_count()) return run_tc<128, 6, EPI_PLAIN>(x, W, out, rows, N, K, 1, partials, logits, n_parts, status, st);
        return run_tc<128, 3, EPI_PLAIN>(x, W, out, rows, N, K, 1, partials, logits, n_parts, status, st);
    }
    if (epi == EPI_SWIGLU) {
        if (tiles < 100) return run_tc<64, 8, EPI_SWIGLU>(x, W, out, rows, N, K, 1, partials, logits, n_parts, status, st);
        if (tiles <= sm_count()) return run_tc<128, 6, EPI_SWIGLU>(x, W, out, rows, N, K, 1, partials, logits, n_parts, status, st);
        return run_tc<128, 3, EPI_SWIGLU>(x, W, out, rows, N, K, 1, partials, logits, n_parts, status, st);
    }
    return cudaErrorInvalidValue;
}

}  // namespace q35
