// Chunkwise gated-linear-attention forward for sm_100a: one persistent kernel.
//
// Work decomposition.  A sequence (one batch b, one head h, T tokens along the scan order)
// is cut into 64-token chunks and the chunks into segments of `cps` chunks.  A work item is
// one (sequence, segment); CTAs take items from an atomic ticket so that an item's
// predecessors are always held by CTAs that already run.  For every segment but the last
// of a sequence the CTA first streams k, g, v only and reduces the segment to an aggregate
// (decay, state increment), publishes it, obtains its incoming state from its predecessors
// by a decoupled look-back, and then streams q, k, g, v once more (k, g, v come from L2) to
// produce the outputs.  Replaces chunk_compute_S_kernel / chunk_scan_*_kernel /
// chunk_fwd_o_kernel of the reference (engine/gtr/backbone/csrc/gla_chunk.cuh:718-1394).
//
// Per chunk, with G the inclusive within-chunk cumulative log gate (fp32, kept in log2
// units), G_m its value at the middle row and G_L at the last row:
//   qh = q*2^G        kh = k*2^(G_L-G)         (fp16, exponents <= 0)
//   qb = qh*2^(-G_m)  kb = kh*2^(G_m-G_L)      (tf32: fp32 range, exponents within +-92)
//   A  = tril(qb kb^T)                 tcgen05.mma kind::tf32  -> TMEM
//   O  = qh S_in + A v                 two tcgen05.mma kind::f16 into one TMEM accumulator
//   S' = 2^(G_L) (.) S_in + kh^T v     tcgen05.mma kind::f16, decay applied in registers (fp32)
// A chunk whose total decay exceeds 2^-92 (e^-64) in any channel takes an exact scalar path for A.
//
// Tensor memory.  An M = 64 accumulator occupies lanes 0-15 of each 32-lane quadrant, so two
// accumulators share the same columns at lane offsets 0 and 16.  A is produced as two N = 32
// halves (key rows 0-31 at lane offset 0, 32-63 at offset 16); O sits at offset 0 and the
// state increment at offset 16 of the same columns.  Every lane of a warp that reads a quadrant
// therefore owns useful data: lanes 0-15 of the warp on quadrant w hold row 16w+l of O (or the left
// half of A), lanes 16-31 hold state row 16w+l-16 (or the right half of A).  Both the score
// accumulator and the output/state accumulator are double-buffered.
//
// Shared memory.  A ring of kNumStages stages of {q, k, g, v} tiles filled by TMA (q and k are
// rewritten in place as qh and kh, the gate tile is reused for the fp16 score tile), two tf32
// operand buffers {qb, kb}, the fp16 copy of the running state, two output tiles and a block of
// barriers and exchange rows.  A stage is handed back to the producer by the completion of the
// chunk's last MMAs (tcgen05.commit on the stage's `empty` barrier), so its lifetime -- which,
// divided by the ring depth, bounds the chunk rate -- does not include the epilogues.
//
// Warp roles: see the comment above gla_fwd_kernel.
#pragma once

#include <type_traits>

#include "gla_device.cuh"

namespace gla {

constexpr int kChunk = 64;
constexpr int kD = 64;                    // K = V = 64
constexpr int kTileBytes = kChunk * 128;  // one fp16 [64 x 64] tile
constexpr int kStageBytes = 4 * kTileBytes;
#ifndef GLA_MIN_CTAS
#define GLA_MIN_CTAS 1
#endif
#ifndef GLA_STAGES
#define GLA_STAGES 4
#endif
constexpr int kCtasPerSm = GLA_MIN_CTAS;    // resident CTAs per SM the launch bounds and the grid size assume
constexpr int kNumStages = GLA_STAGES;
// Five warpgroups of four warps: state group, score group, two gate teams, service warps.
constexpr int kStateWarps = 4, kScoreWarps = 4, kTeamWarps = 4, kGateTeams = 2, kGateWarps = kTeamWarps * kGateTeams;
constexpr int kStateThreads = 32 * kStateWarps, kScoreThreads = 32 * kScoreWarps, kTeamThreads = 32 * kTeamWarps,
              kGateThreads = 32 * kGateWarps;
constexpr int kGateGroups = 8;               // gate math: row groups of eight rows, two per warp of a team
constexpr int kThreads = kStateThreads + kScoreThreads + kGateThreads + 128;
constexpr int kTmemCols = 256;
constexpr uint32_t kTmA = 0;              // scores: two buffers of 32 columns, each two interleaved halves
constexpr uint32_t kTmOS = 64;            // two buffers of 64 columns: outputs (lane offset 0), state increment (lane offset 16)
constexpr int kSlots = 2 * kNumStages;    // per-chunk exchange slots (chunk totals, exact-path flag): outlive the stage
constexpr uint32_t kLane16 = 16u << 16;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kWideLimit = 64.f * kLog2e;   // largest in-chunk decay (log2 units) the tf32 path takes

// tensor ids inside Maps
enum { TQ = 0, TK = 1, TG = 2, TV = 3, TO = 4, TGATE = 5, kNumTensors = 6 };
constexpr int kNumBoxes = 4;              // box heights 64, 16, 4, 1 rows

struct Maps {
    CUtensorMap m[kNumTensors][kNumBoxes];
};

struct Params {
    int B, T, H, NT;
    int K;               // key channels per head, 32 or 64.  A K = 32 head runs as a K = 64 head whose upper 32
                         // channels are zero: the tensor maps of q, k, g give the channel dimension its true extent,
                         // so the TMA loads fill channels 32..63 of every tile with zeros without reading anything,
                         // and state rows 32..63 stay zero
    int Hc, Wc;          // column length / number of columns of the scan (row scans: Hc = T, Wc = 1)
    int rev;             // scan runs from the last token to the first
    int NS, cps;         // segments per sequence, chunks per segment
    int num_items;
    int gated;           // fused RMSNorm * w * silu(gate) epilogue
    // The output scale is folded into the exponent of the q-side gate factors (q_exp = log2(scale), o_mul = 1)
    // when it is positive and finite; otherwise the epilogue multiplies (q_exp = 0, o_mul = scale).
    float q_exp, q_mul, o_mul;
    float inv_norm;      // 1/gk_normalizer, or 0 when g already is a log gate
    float rms_eps;
    const __half* rms_w;      // [64]
    const __half* gate;       // output gate [B,T,H,64] with element strides gate_sb/st/sh
    long long gate_sb, gate_st, gate_sh;
    __half* o;                // output [B,T,H,64] with element strides o_sb/st/sh
    long long o_sb, o_st, o_sh;
    const float* s0;
    float* sT;
    uint32_t* ctrl;      // [0] ticket, [1] status
    uint32_t* flags;     // per (sequence, segment): 0 none, 1 aggregate, 2 inclusive state
    float* agg;          // per (sequence, segment): 4096 state increment + 64 log2 decay
    float* incl;         // per (sequence, segment): 4096 state after the segment
    uint32_t wait_limit_us;
#ifdef GLA_TRACE
    unsigned long long* trace;   // debug builds only: (event, time) pairs of CTA 0
    int dbg;                     // debug builds only: ablation switches (results become wrong)
#endif
};

#ifdef GLA_TRACE
// debug builds: lane 0 of every warp of CTA 0 appends (clock << 8 | event) to its own region, no atomics
#define GLA_EV(id) do { if (blockIdx.x == 0 && !(P.dbg & 128) && (threadIdx.x & 31) == 0 && trace_n < 4096u) { \
        P.trace[(threadIdx.x >> 5) * 4096u + trace_n++] = ((unsigned long long)clock64() << 8) | (unsigned long long)(id); } } while (0)
#define GLA_EVG(id) do { if (blockIdx.x == 0 && (threadIdx.x & 31) == 0 && trace_n < 4096u) { \
        P.trace[(threadIdx.x >> 5) * 4096u + trace_n++] = ((unsigned long long)globaltimer_ns() << 8) | (unsigned long long)(id); } } while (0)
#else
#define GLA_EV(id) do { } while (0)
#define GLA_EVG(id) do { } while (0)
#endif

constexpr int kAggStride = kD * kD + kD;

// shared memory map (bytes from a 1024-aligned base)
constexpr int kOffStage = 0;
constexpr int kOffQbar = kNumStages * kStageBytes;       // two buffers of {qb 16 KB, kb 16 KB} tf32 (each two 8 KB halves)
constexpr int kQkBufBytes = 4 * kTileBytes;
constexpr int kOffKbarRel = 2 * kTileBytes;              // kb inside a buffer
constexpr int kOffS16 = kOffQbar + 2 * kQkBufBytes;
constexpr int kOffOut = kOffS16 + kTileBytes;            // two output tiles (fp16, swizzled), sent out by the store warp
constexpr int kOffMisc = kOffOut + 2 * kTileBytes;
constexpr int kMiscBytes = 8192;
constexpr int kSmemBytes = kOffMisc + kMiscBytes + 1024;  // + alignment slack

struct Misc {
    uint64_t full[kNumStages];
    uint64_t empty[kNumStages];
    // A barrier may run at most one phase ahead of its slowest waiter.  Barriers whose producer can run further
    // ahead are rings indexed like the resource they guard (stage, or tf32 buffer / score accumulator).
    uint64_t o_ready[2], o_free[2], o_norm[2];
    uint64_t ops_ready[kNumStages], a16_ready[kNumStages], a_done[2], a_free[2], os_done[2], os_free[2], s16_ready;
    uint32_t tmem_base;
    volatile uint32_t abort;
    int item;
    uint32_t wide[kSlots];
    alignas(16) float tot[2][kGateGroups][kD];     // gate sums per row group (float4 access), double-buffered
    alignas(16) float b4s[kSlots][kD]; // chunk totals G_L per channel
};
static_assert(sizeof(Misc) <= kMiscBytes, "misc block too large");

enum { WHERE_MBAR = 1, WHERE_LOOKBACK = 2 };

struct Ctx {
    const Params* p;
    Misc* misc;
    uint8_t* base;       // generic pointer to the 1024-aligned shared-memory base
    uint32_t smem;       // the same as a shared-window address
    uint64_t deadline_span_ns;
#ifdef GLA_TRACE
    uint32_t* trace_n;
#endif
};
#if defined(GLA_TRACE) && defined(GLA_TRACE_FINE)
#define GLA_EVC(c, id) do { if (blockIdx.x == 0 && !((c).p->dbg & 128) && (threadIdx.x & 31) == 0 && *(c).trace_n < 4096u) { \
        (c).p->trace[(threadIdx.x >> 5) * 4096u + (*(c).trace_n)++] = ((unsigned long long)clock64() << 8) | (unsigned long long)(id); } } while (0)
#else
#define GLA_EVC(c, id) do { } while (0)
#endif

__device__ __forceinline__ void raise_timeout(const Ctx& c, uint32_t where) {
    c.misc->abort = 1;
    atomicCAS(c.p->ctrl + 1, 0u, where);
}

// Bounded wait.  After a time-out in this CTA every later wait returns at once, so all warps
// keep following the protocol (arrivals, named barriers) and the CTA drains and exits; the
// result is then undefined and the status word says so.
// Every polling thread is on the path of a stage through the pipeline (the stage ring is only kNumStages deep, so
// the time a stage spends between its TMA load and its release bounds the throughput): no sleeping between polls --
// try_wait itself suspends the thread for a while -- and only one warp per group and one lane per single-thread
// role ever polls.
#ifndef GLA_SPIN_SLEEP_NS
#define GLA_SPIN_SLEEP_NS 0
#endif
__device__ __forceinline__ void mbar_wait_slow(const Ctx& c, uint32_t b, uint32_t parity) {
    const uint64_t t0 = globaltimer_ns();
    uint32_t n = 0;
    while (true) {
        if (mbar_try_wait(b, parity)) return;
        if (GLA_SPIN_SLEEP_NS > 0) __nanosleep(GLA_SPIN_SLEEP_NS);
        if ((++n & 255u) == 0u) {
            if (c.misc->abort) return;
            if (globaltimer_ns() - t0 > c.deadline_span_ns) {
                raise_timeout(c, WHERE_MBAR);
                return;
            }
        }
    }
}
__device__ __forceinline__ void mbar_wait(const Ctx& c, uint64_t* bar, uint32_t parity) {
    const uint32_t b = smem_u32(bar);
    if (mbar_try_wait(b, parity)) return;
    mbar_wait_slow(c, b, parity);
}

// Wait of a whole warp group: its first warp polls the mbarrier, the others sleep in the hardware barrier
// `bar_id` (a warp parked in bar.sync issues nothing, a polling warp competes with the working ones).
__device__ __forceinline__ void group_wait(const Ctx& c, uint64_t* bar, uint32_t parity, int group_warp, uint32_t bar_id,
                                           uint32_t group_threads) {
    if (group_warp == 0) mbar_wait(c, bar, parity);
    named_bar_sync(bar_id, group_threads);
}

// One arrival per warp: the lanes order their work before lane 0 with a warp barrier, lane 0 arrives for all of
// them.  (Per-thread arrivals are 32 serialized updates of one shared-memory word per warp.)
__device__ __forceinline__ void warp_arrive(uint64_t* bar, int lane) {
    __syncwarp();
    if (lane == 0) mbar_arrive(smem_u32(bar));
}

// Walks the chunks of one pass along the scan and enumerates, for the current chunk, the TMA boxes that cover
// it: f(box_id, r, c, smem_row) with (r, c) the row inside the column and the column where the box starts.  The
// position is advanced chunk by chunk, so the loop needs no division.
struct BoxWalker {
    int u_lo;     // scan position of the chunk's first row (may be negative for the ragged chunk of a reversed scan)
    int c, r;     // column and row inside the column of max(u_lo, 0)
    __device__ __forceinline__ BoxWalker(const Params& P, int p0) {
        u_lo = P.rev ? (P.T - p0 - kChunk) : p0;
        const int u0 = max(u_lo, 0);
        c = u0 / P.Hc;
        r = u0 - c * P.Hc;
    }
    template <class F>
    __device__ __forceinline__ void for_each(const Params& P, F f) const {
        int u0 = max(u_lo, 0);
        const int u1 = min(u_lo + kChunk, P.T);
        int cc = c, rr = r;
        while (u0 < u1) {
            int len = min(P.Hc - rr, u1 - u0);
            while (len > 0) {
                const int id = len >= 64 ? 0 : len >= 16 ? 1 : len >= 4 ? 2 : 3;
                const int R = 64 >> (2 * id);
                f(id, rr, cc, u0 - u_lo);
                rr += R;
                u0 += R;
                len -= R;
            }
            if (rr >= P.Hc) { rr = 0; ++cc; }
        }
    }
    __device__ __forceinline__ void advance(const Params& P) {
        if (!P.rev) {
            u_lo += kChunk;
            r += kChunk;
            while (r >= P.Hc) { r -= P.Hc; ++c; }
        } else {
            u_lo -= kChunk;
            if (u_lo >= 0) {
                r -= kChunk;
                while (r < 0) { r += P.Hc; --c; }
            } else {
                c = 0;
                r = 0;
            }
        }
    }
};

__device__ __forceinline__ int chunk_valid(int p0, int L) { return min(kChunk, L - p0); }

// Shared memory is always addressed through the shared window (ld.shared / st.shared): generic
// loads of shared data take the slow path through L1TEX.
__device__ __forceinline__ uint32_t lds32(uint32_t a) { return ld_shared_u32(a); }
__device__ __forceinline__ void sts32(uint32_t a, uint32_t v) { st_shared_u32(a, v); }
__device__ __forceinline__ void sts64(uint32_t a, float x, float y) { st_shared_f2(a, x, y); }

// ------------------------------------------------------------------------------------------
#ifdef GLA_TRACE
#define GLA_DBG(bit) ((c.p->dbg >> (bit)) & 1)
#define GLA_DBGP(bit) ((P.dbg >> (bit)) & 1)
#else
#define GLA_DBG(bit) 0
#define GLA_DBGP(bit) 0
#endif
// Gate math for one chunk (the four warps of one gate team; `bar_id` is the team's named barrier).  Thread (w, l) owns the eight logical rows
// 16w + 8(l>>4) .. +7 (row group 2w + (l>>4)) and the four channels 4(l&15) .. +3, so that every access is a
// 64-bit (fp16 tiles) or 128-bit (tf32 tiles, exchange rows) shared-memory instruction.  Logical row =
// position inside the chunk along the scan; the physical (shared-memory / TMEM) row is mirrored for reversed
// scans.  Tiles are rows of 128 bytes whose 16-byte units are XOR-swizzled with (row & 7); a thread's first row
// is a multiple of 8, so the swizzle of its i-th row depends on i only, a compile-time constant here.
//
// The row loops are rolled (two to four rows per iteration, the running gate sum carried in registers and the
// gate tile read a second time after the exchange): fully unrolled, the gate math alone was 50 KB of straight-line
// code that every warp streamed through the instruction caches once per chunk, and instruction fetch was the
// second largest stall of the kernel.  Ragged chunks and chunks on the exact path take out-of-line versions.
struct GateLane {
    uint32_t a16;    // byte offset of (first logical row, first channel) in an fp16 tile, without the swizzle term
    uint32_t a32;    // same for the two-half tf32 tiles
    uint32_t x16;    // swizzle term (16-byte unit index << 4) of the first row, fp16 tiles
    uint32_t x32;    // same, tf32 tiles
};
template <bool kRev>
__device__ __forceinline__ GateLane gate_lane(int w, int l) {
    GateLane g;
    const uint32_t cg = l & 15u;                                    // channel group: channels 4cg .. 4cg+3
    const uint32_t first = 16u * w + 8u * (l >> 4);                 // first logical row, a multiple of 8
    const uint32_t row0 = kRev ? (63u - first) : first;
    // (physical row & 7) of logical row first + i is i forward and 7 - i = 7 ^ i reversed
    const uint32_t rbits = kRev ? 7u : 0u;
    g.a16 = row0 * 128u + ((cg & 1u) << 3);
    g.a32 = row0 * 128u + (cg >> 3) * kTileBytes;
    g.x16 = ((cg >> 1) ^ rbits) << 4;
    g.x32 = ((cg & 7u) ^ rbits) << 4;
    return g;
}
// offsets of the thread's i-th row (i is a compile-time constant at every use in the hot path)
template <bool kRev> __device__ __forceinline__ uint32_t off16(const GateLane& g, int i) {
    return (kRev ? g.a16 - 128u * i : g.a16 + 128u * i) + (g.x16 ^ (static_cast<uint32_t>(i) << 4));
}
template <bool kRev> __device__ __forceinline__ uint32_t off32(const GateLane& g, int i) {
    return (kRev ? g.a32 - 128u * i : g.a32 + 128u * i) + (g.x32 ^ (static_cast<uint32_t>(i) << 4));
}
__device__ __forceinline__ void unpack4(uint2 r, float* x) {
    const float2 a = unpack_half2(r.x), b = unpack_half2(r.y);
    x[0] = a.x; x[1] = a.y; x[2] = b.x; x[3] = b.y;
}

struct Gate4 { float v[4]; };
#define GLA_PRAGMA_(x) _Pragma(#x)
#define GLA_PRAGMA_UNROLL(n) GLA_PRAGMA_(unroll n)
#ifndef GLA_GATE_UNROLL_A
#define GLA_GATE_UNROLL_A 4
#endif
#ifndef GLA_GATE_UNROLL_B
#define GLA_GATE_UNROLL_B 2
#endif

// Rolled, out-of-line row pass for the rare cases: a ragged last chunk (rows past `valid` are zeroed)
// and chunks on the exact-score path (`wide`: G and raw q, k are stashed in plain layouts where the
// tf32 operands would go).  Recomputes the running gate sum from the (still raw) gate tile.
template <bool kRev>
__device__ __noinline__ void gate_rows_general(const Ctx& c, uint32_t stage, uint32_t qbar, int valid, int w, int l,
                                               bool state_only, bool wide, Gate4 off, Gate4 b4, Gate4 e1, Gate4 e2) {
    const float qx = c.p->q_exp;
    const GateLane gl = gate_lane<kRev>(w, l);
    const uint32_t tq = stage, tk = stage + kTileBytes, tg = stage + 2 * kTileBytes, tv = stage + 3 * kTileBytes;
    const uint32_t kbar = qbar + kOffKbarRel;
    const uint32_t c0 = 4u * (l & 15u);
    const int first = 16 * w + 8 * (l >> 4);
    float a[4] = {off.v[0], off.v[1], off.v[2], off.v[3]};
#pragma unroll 1
    for (int i = 0; i < 8; ++i) {
        const uint32_t o16 = (kRev ? gl.a16 - 128u * i : gl.a16 + 128u * i) + (gl.x16 ^ (static_cast<uint32_t>(i) << 4));
        const uint32_t o32 = (kRev ? gl.a32 - 128u * i : gl.a32 + 128u * i) + (gl.x32 ^ (static_cast<uint32_t>(i) << 4));
        const bool live = first + i < valid;
        float gv[4], kv[4], qv[4], kh[4], qh[4];
        unpack4(ld_shared_v2(tg + o16), gv);
        const uint2 kr = live ? ld_shared_v2(tk + o16) : make_uint2(0u, 0u);
        const uint2 qr = (live && !state_only) ? ld_shared_v2(tq + o16) : make_uint2(0u, 0u);
        unpack4(kr, kv);
        unpack4(qr, qv);
#pragma unroll
        for (int ch = 0; ch < 4; ++ch) {
            a[ch] += live ? gv[ch] * kLog2e : 0.f;
            kh[ch] = kv[ch] * ex2(b4.v[ch] - a[ch]);
            qh[ch] = qv[ch] * ex2(a[ch] + qx);
        }
        st_shared_v2(tk + o16, pack_half2_sat(kh[0], kh[1]), pack_half2_sat(kh[2], kh[3]));
        if (!live) st_shared_v2(tv + o16, 0u, 0u);                // rows past the end must be finite for the MMAs
        if (!state_only) {
            st_shared_v2(tq + o16, pack_half2_sat(qh[0], qh[1]), pack_half2_sat(qh[2], qh[3]));
            if (!wide) {
                st_shared_f4(qbar + o32, round_tf32(qh[0] * e1.v[0]), round_tf32(qh[1] * e1.v[1]),
                             round_tf32(qh[2] * e1.v[2]), round_tf32(qh[3] * e1.v[3]));
                st_shared_f4(kbar + o32, round_tf32(kh[0] * e2.v[0]), round_tf32(kh[1] * e2.v[1]),
                             round_tf32(kh[2] * e2.v[2]), round_tf32(kh[3] * e2.v[3]));
            } else {   // plain layouts: G fp32 [64][64] at qbar; raw q, k fp16 [64][64] at kbar
                const int rho = kRev ? 63 - (first + i) : first + i;
                st_shared_f4(qbar + rho * 256 + c0 * 4, a[0], a[1], a[2], a[3]);
                st_shared_v2(kbar + rho * 128 + c0 * 2, qr.x, qr.y);
                st_shared_v2(kbar + kTileBytes + rho * 128 + c0 * 2, kr.x, kr.y);
            }
        }
    }
}

template <bool kStateOnly, bool kRev, bool kLogits>
__device__ __forceinline__ bool gate_math_t(const Ctx& c, uint32_t stage, uint32_t qbar, int n, int valid, int w, int l,
                                            uint64_t* buf_bar, uint32_t buf_parity, uint32_t bar_id) {
    constexpr int R = 8;
    const Params& P = *c.p;
    Misc& M = *c.misc;
    const int par = n & 1, slot = n % kSlots;
    const GateLane gl = gate_lane<kRev>(w, l);
    const uint32_t tq = stage, tk = stage + kTileBytes, tg = stage + 2 * kTileBytes;
    const uint32_t kbar = qbar + kOffKbarRel;
    const uint32_t c0 = 4u * (l & 15u);
    const int grp = 2 * w + (l >> 4);                        // row group (eight rows) of this thread
    const uint32_t tot_sa = smem_u32(&M.tot[par][0][c0]);   // + group * kD * 4
    const bool ragged = valid < kChunk;

    GLA_EVC(c, 45);
    {
        float a[4] = {0.f, 0.f, 0.f, 0.f};
        const float inv_norm = P.inv_norm;
        GLA_PRAGMA_UNROLL(GLA_GATE_UNROLL_A)
        for (int i = 0; i < R; ++i) {
            float gv[4];
            unpack4(ld_shared_v2(tg + off16<kRev>(gl, i)), gv);
            if constexpr (kLogits) {
                // raw-logit gates (gk_normalizer > 0): the tile is rewritten in place as fp16 log gates,
                // logsigmoid(x) / normalizer; each thread converts the rows it owns and reads only those later
                const uint32_t h0 = pack_half2_sat(logsigmoid_f(gv[0]) * inv_norm, logsigmoid_f(gv[1]) * inv_norm);
                const uint32_t h1 = pack_half2_sat(logsigmoid_f(gv[2]) * inv_norm, logsigmoid_f(gv[3]) * inv_norm);
                st_shared_v2(tg + off16<kRev>(gl, i), h0, h1);
                unpack4(make_uint2(h0, h1), gv);
            }
            const bool live = 16 * w + 8 * (l >> 4) + i < valid;
#pragma unroll
            for (int ch = 0; ch < 4; ++ch) a[ch] = fmaf(live ? gv[ch] : 0.f, kLog2e, a[ch]);
        }
        st_shared_f4(tot_sa + grp * kD * 4, a[0], a[1], a[2], a[3]);
    }
    GLA_EVC(c, 40);
    // the tf32 buffer written below is free once the score MMAs of its previous use have completed; one warp
    // polls for that, the exchange barrier tells the others
    if (!kStateOnly && w == 0) mbar_wait(c, buf_bar, buf_parity);
    named_bar_sync(bar_id, kTeamThreads);
    GLA_EVC(c, 41);
    Gate4 off, b4, gm;
#pragma unroll
    for (int ch = 0; ch < 4; ++ch) off.v[ch] = b4.v[ch] = gm.v[ch] = 0.f;
#pragma unroll
    for (int g = 0; g < kGateGroups; ++g) {
        const float4 t4 = ld_shared_f4(tot_sa + g * kD * 4);
        const float t[4] = {t4.x, t4.y, t4.z, t4.w};
#pragma unroll
        for (int ch = 0; ch < 4; ++ch) {
            if (g < grp) off.v[ch] += t[ch];
            if (g == kGateGroups / 2) gm.v[ch] = b4.v[ch];      // sum of the first half: the mid-chunk reference
            b4.v[ch] += t[ch];
        }
    }
    if (grp == 0) st_shared_f4(smem_u32(&M.b4s[slot][c0]), b4.v[0], b4.v[1], b4.v[2], b4.v[3]);
    bool wide = false;
    Gate4 e1, e2;
#pragma unroll
    for (int ch = 0; ch < 4; ++ch) e1.v[ch] = e2.v[ch] = 0.f;
    if (!kStateOnly) {
        wide = __any_sync(0xffffffffu, (-b4.v[0] > kWideLimit) || (-b4.v[1] > kWideLimit) || (-b4.v[2] > kWideLimit) ||
                                           (-b4.v[3] > kWideLimit));
        if (w == 0 && l == 0) M.wide[slot] = wide ? 1u : 0u;
#pragma unroll
        for (int ch = 0; ch < 4; ++ch) {
            e1.v[ch] = ex2(-gm.v[ch]);
            e2.v[ch] = ex2(gm.v[ch] - b4.v[ch]);
        }
    }
    if (ragged || wide) {
        gate_rows_general<kRev>(c, stage, qbar, valid, w, l, kStateOnly, wide, off, b4, e1, e2);
    } else {
        float r[4] = {off.v[0], off.v[1], off.v[2], off.v[3]};   // running inclusive gate sum of the current row
        const float qx = P.q_exp;
        GLA_PRAGMA_UNROLL(GLA_GATE_UNROLL_B)
        for (int i = 0; i < R; ++i) {
            float gv[4], kv[4], kh[4];
            unpack4(ld_shared_v2(tg + off16<kRev>(gl, i)), gv);
            unpack4(ld_shared_v2(tk + off16<kRev>(gl, i)), kv);
#pragma unroll
            for (int ch = 0; ch < 4; ++ch) {
                r[ch] = fmaf(gv[ch], kLog2e, r[ch]);
                kh[ch] = kv[ch] * ex2(b4.v[ch] - r[ch]);
            }
            st_shared_v2(tk + off16<kRev>(gl, i), pack_half2(kh[0], kh[1]), pack_half2(kh[2], kh[3]));
            if (!kStateOnly) {
                float qv[4], qh[4];
                unpack4(ld_shared_v2(tq + off16<kRev>(gl, i)), qv);
#pragma unroll
                for (int ch = 0; ch < 4; ++ch) qh[ch] = qv[ch] * ex2(r[ch] + qx);
                st_shared_v2(tq + off16<kRev>(gl, i), pack_half2(qh[0], qh[1]), pack_half2(qh[2], qh[3]));
                st_shared_f4(qbar + off32<kRev>(gl, i), round_tf32(qh[0] * e1.v[0]), round_tf32(qh[1] * e1.v[1]),
                             round_tf32(qh[2] * e1.v[2]), round_tf32(qh[3] * e1.v[3]));
                st_shared_f4(kbar + off32<kRev>(gl, i), round_tf32(kh[0] * e2.v[0]), round_tf32(kh[1] * e2.v[1]),
                             round_tf32(kh[2] * e2.v[2]), round_tf32(kh[3] * e2.v[3]));
            }
        }
    }
    GLA_EVC(c, 42);
    fence_proxy_async_smem();
    GLA_EVC(c, 43);
    return wide;
}

// Returns whether the chunk took the exact-score path (always false for state-only chunks).
__device__ __forceinline__ bool gate_math(const Ctx& c, uint32_t stage, uint32_t qbar, int n, int valid, int w, int l,
                                          bool state_only, uint64_t* buf_bar, uint32_t buf_parity, uint32_t bar_id) {
    // one instantiation per (pass, scan direction, gate kind): a launch runs two of them, and the others cost it
    // neither registers nor instruction-cache space
    const bool logits = c.p->inv_norm > 0.f;
#define GLA_GATE_CALL(SO, RV, LG) gate_math_t<SO, RV, LG>(c, stage, qbar, n, valid, w, l, buf_bar, buf_parity, bar_id)
    if (c.p->rev) {
        if (state_only) return logits ? GLA_GATE_CALL(true, true, true) : GLA_GATE_CALL(true, true, false);
        return logits ? GLA_GATE_CALL(false, true, true) : GLA_GATE_CALL(false, true, false);
    }
    if (state_only) return logits ? GLA_GATE_CALL(true, false, true) : GLA_GATE_CALL(true, false, false);
    return logits ? GLA_GATE_CALL(false, false, true) : GLA_GATE_CALL(false, false, false);
#undef GLA_GATE_CALL
}

__device__ __forceinline__ uint32_t sw_f16(uint32_t row, uint32_t col) {     // col in fp16 elements
    return row * 128u + ((((col >> 3) ^ row) & 7u) << 4) + ((col & 7u) << 1);
}

// Exact intra-chunk scores for chunks whose gates are too strong for a common reference:
// A[i][j] = sum_c q[i][c] k[j][c] 2^(G[i][c] - G[j][c]) for j at or before i along the scan.
__device__ __noinline__ void exact_scores(const Ctx& c, uint8_t* a16_tile, const uint8_t* qkbuf, int tid, int nthreads) {
    const bool rev = c.p->rev != 0;
    const uint8_t* gs = qkbuf;
    const uint8_t* qs = qkbuf + kOffKbarRel;
    const uint8_t* ks = qs + kTileBytes;
    const uint32_t kPerRow = static_cast<uint32_t>(nthreads) / kChunk;
    const uint32_t i = tid / kPerRow;
    for (uint32_t j = tid % kPerRow; j < 64; j += kPerRow) {
        float s = 0.f;
        const bool keep = rev ? (j >= i) : (j <= i);
        if (keep) {
            for (uint32_t ch = 0; ch < 64; ch += 2) {
                const float2 gi = *reinterpret_cast<const float2*>(gs + i * 256u + ch * 4u);
                const float2 gj = *reinterpret_cast<const float2*>(gs + j * 256u + ch * 4u);
                const float2 qv = unpack_half2(*reinterpret_cast<const uint32_t*>(qs + i * 128u + ch * 2u));
                const float2 kv = unpack_half2(*reinterpret_cast<const uint32_t*>(ks + j * 128u + ch * 2u));
                s += qv.x * kv.x * ex2(gi.x - gj.x);
                s += qv.y * kv.y * ex2(gi.y - gj.y);
            }
        }
        s *= c.p->q_mul;
        const __half hv = __float2half_rn(fminf(fmaxf(s, -65504.f), 65504.f));
        *reinterpret_cast<__half*>(a16_tile + sw_f16(i, j)) = hv;
    }
}

// Read `N` consecutive fp32 columns of this thread's TMEM lane (N = 32 or 64).
template <int N>
__device__ __forceinline__ void tmem_row(uint32_t tmem_base, int w, uint32_t col, float* x) {
    const uint32_t addr = tmem_base + (static_cast<uint32_t>(32 * w) << 16) + col;
    uint32_t* r = reinterpret_cast<uint32_t*>(x);
    __syncwarp();   // tcgen05.ld is warp-collective; lane 0 may come from a single-thread branch
    if constexpr (N == 8) {
        tmem_ld8(addr, r);
    } else {
#pragma unroll
        for (int k = 0; k < N / 16; ++k) tmem_ld16(addr + 16 * k, r + 16 * k);
    }
    tmem_ld_wait();
}

// Write 8*N8 floats as fp16 into 16-byte units unit0.. of one row of a swizzled tile.
template <int N8>
__device__ __forceinline__ void store_row_f16(uint32_t tile, uint32_t row, uint32_t unit0, const float* x) {
#pragma unroll
    for (uint32_t m = 0; m < N8; ++m) {
        const uint32_t a = tile + row * 128u + ((((unit0 + m) ^ row) & 7u) << 4);
        st_shared_v4(a, pack_half2(x[8 * m], x[8 * m + 1]), pack_half2(x[8 * m + 2], x[8 * m + 3]),
                     pack_half2(x[8 * m + 4], x[8 * m + 5]), pack_half2(x[8 * m + 6], x[8 * m + 7]));
    }
}

// Causal mask along the scan on N score columns j0.. of query row rho (keep key j0 + j at or before the query;
// at or after it for reversed scans), then the fp16 tile.  Branch-free selects: the two half-warps sit on
// different sides of the diagonal.
template <int N>
__device__ __forceinline__ void mask_and_store_scores(bool rev, uint32_t a16, uint32_t rho, uint32_t j0, float* x) {
    const int lim = static_cast<int>(rho) - static_cast<int>(j0);
    if (!rev) {
#pragma unroll
        for (int j = 0; j < N; ++j) x[j] = (j <= lim) ? x[j] : 0.f;
    } else {
#pragma unroll
        for (int j = 0; j < N; ++j) x[j] = (j >= lim) ? x[j] : 0.f;
    }
    store_row_f16<N / 8>(a16, rho, j0 >> 3, x);
}

// Self-test of the bounded waits: one warp waits on an mbarrier nobody arrives at and on a global
// flag nobody sets.  Both waits must give up after the limit, set the status word and return.
__global__ void wait_timeout_selftest_kernel(Params P) {
    __shared__ Misc M;
    Ctx ctx;
    ctx.p = &P;
    ctx.misc = &M;
    ctx.base = nullptr;
    ctx.smem = 0;
    ctx.deadline_span_ns = static_cast<uint64_t>(P.wait_limit_us) * 1000ull;
#ifdef GLA_TRACE
    uint32_t trace_n = 0;
    ctx.trace_n = &trace_n;
#endif
    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&M.full[0]), 1);
        M.abort = 0;
        fence_mbar_init();
    }
    __syncthreads();
    mbar_wait(ctx, &M.full[0], 0);                 // never completes: returns after the limit
    const uint64_t t0 = globaltimer_ns();
    while (ld_acquire_gpu(P.flags) == 0u) {        // never set: same exit rule as the look-back
        if (globaltimer_ns() - t0 > ctx.deadline_span_ns) {
            raise_timeout(ctx, WHERE_LOOKBACK);
            break;
        }
        __nanosleep(64);
    }
    __syncthreads();
    if (threadIdx.x == 0) P.ctrl[2] = M.abort;     // 1: the CTA noticed the time-out
}

struct ItemInfo {
    int seq, seg, b, h, first_chunk, nchunks, state_pass;
};

__device__ __forceinline__ ItemInfo decode_item(const Params& P, int item) {
    ItemInfo it;
    const int nseq = P.B * P.H;
    it.seg = item / nseq;
    it.seq = item - it.seg * nseq;
    it.b = it.seq / P.H;
    it.h = it.seq - it.b * P.H;
    it.first_chunk = it.seg * P.cps;
    it.nchunks = min(P.cps, P.NT - it.first_chunk);
    it.state_pass = (it.seg < P.NS - 1) ? 1 : 0;
    return it;
}

// Warp roles (one CTA per SM, 20 warps in five warpgroups):
//   warps 0..3   state group    TMEM read-out of outputs and state increments: state in fp32 registers (lanes
//                               16-31: one state row each; lanes 0-15: one output row each), fp16 copy of the state
//                               for the next chunk, output tile, look-back and publication of segment states
//   warps 4..7   score group    TMEM read-out of the intra-chunk scores -> causal mask -> fp16 tile
//   warps 8..15  gate group     raw q,k,g tiles -> qh, kh (fp16, in place) and qb, kb (tf32, two buffers); two
//                               teams of four warps that take the chunks in turn
//   warp 16      TMA producer   warp 17  score MMAs   warp 18  output and state MMAs   warp 19  output TMA stores
// The chain from one chunk's state to the next (state group -> output MMAs -> state group) is the serial part of a
// sequence, and everything on it is a dependent sequence of synchronising operations that cost tens of cycles each;
// the score read-out is therefore a group of its own and overlaps it.  The gate group is throughput work and runs
// up to two chunks ahead (bounded by the tf32 buffers).  Each warpgroup sets its own register budget (setmaxnreg):
// the state group holds a 64-wide state row per thread, the four service warps need next to nothing.
//
// Register budgets per thread of the five warpgroups.  setmaxnreg only re-divides what the CTA got at launch
// (kThreads x the kernel's register count, 96 under these launch bounds), and an increase waits, without limit, until
// the other groups have released enough: the budgets must not add up to more than that.
#ifndef GLA_REGS_STATE
#define GLA_REGS_STATE 152
#define GLA_REGS_SCORE 64
#define GLA_REGS_GATE 112
#define GLA_REGS_SERVICE 40
#endif
constexpr int kRegsState = GLA_REGS_STATE, kRegsScore = GLA_REGS_SCORE, kRegsGate = GLA_REGS_GATE, kRegsService = GLA_REGS_SERVICE;
constexpr int kLaunchRegs = 96;
constexpr int kRegBudgetTotal = kStateThreads * kRegsState + kScoreThreads * kRegsScore + kGateThreads * kRegsGate + 128 * kRegsService;
#ifndef GLA_REGS_NOCHECK
static_assert(kRegBudgetTotal <= kThreads * kLaunchRegs, "register budgets exceed what the CTA is launched with");
#endif

__global__ void __launch_bounds__(kThreads, kCtasPerSm)
gla_fwd_kernel(const __grid_constant__ Maps maps, const __grid_constant__ Params P) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t* base_ptr = smem_raw + (base - raw);
    Misc& M = *reinterpret_cast<Misc*>(base_ptr + kOffMisc);

    const int tid = threadIdx.x;
    const int w = tid >> 5, l = tid & 31;
#ifdef GLA_TRACE
    uint32_t trace_n = 0;
#endif
    constexpr int kWarpGate = kStateWarps + kScoreWarps;
    constexpr int kWarpProducer = kWarpGate + kGateWarps, kWarpMma = kWarpProducer + 1;

    Ctx ctx;
    ctx.p = &P;
    ctx.misc = &M;
    ctx.base = base_ptr;
    ctx.smem = base;
    ctx.deadline_span_ns = static_cast<uint64_t>(P.wait_limit_us) * 1000ull;
#ifdef GLA_TRACE
    ctx.trace_n = &trace_n;
#endif

    if (tid == 0) {
        for (int s = 0; s < kNumStages; ++s) {
            mbar_init(smem_u32(&M.full[s]), 1);
            mbar_init(smem_u32(&M.empty[s]), 1);
            mbar_init(smem_u32(&M.ops_ready[s]), kTeamWarps);
            mbar_init(smem_u32(&M.a16_ready[s]), kScoreWarps);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(smem_u32(&M.a_done[b]), 1);
            mbar_init(smem_u32(&M.a_free[b]), kScoreWarps);
            mbar_init(smem_u32(&M.os_done[b]), 1);
            mbar_init(smem_u32(&M.os_free[b]), kStateWarps);
            mbar_init(smem_u32(&M.o_ready[b]), kStateWarps);
            mbar_init(smem_u32(&M.o_free[b]), 1);
            mbar_init(smem_u32(&M.o_norm[b]), kStateWarps);
        }
        mbar_init(smem_u32(&M.s16_ready), kStateWarps);
        M.abort = 0;
#ifdef GLA_TRACE
        for (int i = 0; i < kSlots; ++i) M.wide[i] = 0;
#endif
        fence_mbar_init();
    }
    if (w == kWarpProducer) {
        tmem_alloc(smem_u32(&M.tmem_base), kTmemCols);
        tmem_relinquish();
    }
    if (w == kWarpMma && l == 0) {
        for (int t = 0; t < TGATE; ++t) tma_prefetch_desc(&maps.m[t][0]);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = __shfl_sync(0xffffffffu, M.tmem_base, 0);

    // Every role walks the same sequence of work items and chunks and keeps its own counters:
    //   ctr  chunks seen so far (both passes): stage = ctr % kNumStages, exchange slot = ctr % kSlots
    //   c2   output-pass chunks seen so far: tf32 buffer / score accumulator / output tile = c2 & 1
    uint32_t ctr = 0, c2 = 0;
    // Work items come from a ticket counter; all roles fetch the same item at the same two block barriers.
    auto next_item = [&]() -> int {
        if (tid == 0) M.item = static_cast<int>(atomicAdd(P.ctrl, 1u));
        __syncthreads();
        return __shfl_sync(0xffffffffu, M.item, 0);   // known to be warp-uniform
    };

    if (w < kStateWarps) {
        // ==================================================================== state group
        reg_alloc<kRegsState>();
        const int etid = tid;
        const bool owner = l >= 16;
        const int quad = w;
        const int my_c = 16 * quad + (l & 15);          // state row (channel) of lanes 16-31
        const uint32_t rho = 16 * quad + (l & 15);      // output row of lanes 0-15
        float S[kD];
        GLA_EV(62);
        GLA_EVG(60);
        while (true) {
            const int item = next_item();
            if (item >= P.num_items) break;
            const ItemInfo it = decode_item(P, item);
            const int npass = it.state_pass ? 2 : 1;
            const size_t srow = (static_cast<size_t>(it.seq) * P.K + my_c) * kD;   // this thread's state row
            const bool real_row = my_c < P.K;      // rows of channels a K = 32 head does not have are zero throughout
            const size_t slot = static_cast<size_t>(it.seq) * P.NS + it.seg;
            float gsum = 0.f;       // log2 of the segment's total decay for channel my_c

            auto load_initial = [&]() {
#pragma unroll
                for (int x = 0; x < kD; ++x) S[x] = 0.f;
                if (owner && real_row && P.s0 != nullptr) {
                    const float4* src = reinterpret_cast<const float4*>(P.s0 + srow);
#pragma unroll
                    for (int x = 0; x < kD / 4; ++x) {
                        const float4 v4 = __ldg(src + x);
                        S[4 * x] = v4.x; S[4 * x + 1] = v4.y; S[4 * x + 2] = v4.z; S[4 * x + 3] = v4.w;
                    }
                }
            };
            auto publish = [&](float* dst_row, uint32_t flag_value) {
                if (owner) {
                    float4* dst = reinterpret_cast<float4*>(dst_row);
#pragma unroll
                    for (int x4 = 0; x4 < kD / 4; ++x4)
                        dst[x4] = make_float4(S[4 * x4], S[4 * x4 + 1], S[4 * x4 + 2], S[4 * x4 + 3]);
                }
                // The group barrier orders every thread's stores before thread 0's release store, and a release is
                // cumulative over what its thread has synchronised with: no per-thread fence is needed (a
                // sequentially-consistent fence per thread costs microseconds under full memory load).
                named_bar_sync(2, kStateThreads);
                if (etid == 0) st_release_gpu(P.flags + slot, flag_value);
            };

            for (int pass = 0; pass < npass; ++pass) {
                const bool state_only = it.state_pass && pass == 0;
                if (state_only) {
                    // pass 1 reduces the segment to (decay, increment); segment 0 folds the initial state in
                    if (it.seg == 0) load_initial();
                    else {
#pragma unroll
                        for (int x = 0; x < kD; ++x) S[x] = 0.f;
                    }
                } else {
                    if (it.seg == 0) load_initial();
                    else {
                        // decoupled look-back: S <- state entering this segment
#pragma unroll
                        for (int x = 0; x < kD; ++x) S[x] = 0.f;
                        float dlog = 0.f;
                        int j = it.seg - 1;
                        const uint64_t t0 = globaltimer_ns();
                        while (true) {
                            const size_t sj = static_cast<size_t>(it.seq) * P.NS + j;
                            // one lane per warp polls (the CTAs of later segments wait here for a whole pre-pass of
                            // their predecessors: 128 polling threads each would only load the L2), the warp barrier of
                            // the shuffle passes the acquired view on to the other lanes
                            uint32_t f = 0u;
                            if (l == 0) {
                                f = ld_acquire_gpu(P.flags + sj);
                                for (uint32_t n = 1; f == 0u; ++n) {
                                    if ((n & 15u) == 0u) {
                                        if (M.abort || ld_acquire_gpu(P.ctrl + 1) != 0u) break;
                                        if (globaltimer_ns() - t0 > ctx.deadline_span_ns) {
                                            raise_timeout(ctx, WHERE_LOOKBACK);
                                            break;
                                        }
                                    }
                                    __nanosleep(128);
                                    f = ld_acquire_gpu(P.flags + sj);
                                }
                            }
                            f = __shfl_sync(0xffffffffu, f, 0);
                            const bool gave_up = f == 0u;
                            const bool inclusive = f == 2u;
                            if (gave_up) break;   // result undefined, status word set
                            const float dacc = ex2(dlog);
                            const float* src_row = inclusive ? P.incl + sj * (kD * kD) + my_c * kD
                                                             : P.agg + sj * kAggStride + my_c * kD;
                            if (owner) {
                                const float4* src = reinterpret_cast<const float4*>(src_row);
#pragma unroll
                                for (int x4 = 0; x4 < kD / 4; ++x4) {
                                    const float4 v4 = __ldcg(src + x4);
                                    S[4 * x4] = fmaf(dacc, v4.x, S[4 * x4]);
                                    S[4 * x4 + 1] = fmaf(dacc, v4.y, S[4 * x4 + 1]);
                                    S[4 * x4 + 2] = fmaf(dacc, v4.z, S[4 * x4 + 2]);
                                    S[4 * x4 + 3] = fmaf(dacc, v4.w, S[4 * x4 + 3]);
                                }
                                if (!inclusive) dlog += __ldcg(P.agg + sj * kAggStride + kD * kD + my_c);
                            }
                            if (inclusive) break;
                            --j;   // never drops below 0: segment 0 only ever publishes an inclusive state
                            if (j < 0) break;
                        }
                        if (it.state_pass) {
                            // inclusive state after this segment = decay * incoming + increment
                            if (owner) {
                                const float dseg = ex2(gsum);
                                const float4* inc = reinterpret_cast<const float4*>(P.agg + slot * kAggStride + my_c * kD);
                                float4* dst = reinterpret_cast<float4*>(P.incl + slot * (kD * kD) + my_c * kD);
#pragma unroll
                                for (int x4 = 0; x4 < kD / 4; ++x4) {
                                    const float4 a4 = __ldcg(inc + x4);
                                    dst[x4] = make_float4(fmaf(dseg, S[4 * x4], a4.x), fmaf(dseg, S[4 * x4 + 1], a4.y),
                                                          fmaf(dseg, S[4 * x4 + 2], a4.z), fmaf(dseg, S[4 * x4 + 3], a4.w));
                                }
                            }
                            named_bar_sync(2, kStateThreads);
                            if (etid == 0) st_release_gpu(P.flags + slot, 2u);
                        }
                    }
                    if (owner) store_row_f16<kD / 8>(base + kOffS16, rho, 0, S);
                    fence_proxy_async_smem();
                    warp_arrive(&M.s16_ready, l);
                }

                // two instantiations of the chunk loop: the fused epilogue's code must not weigh on the plain operator
                auto run_chunks = [&](auto gated_tag) {
                constexpr bool kGated = decltype(gated_tag)::value;
                for (int i = 0; i < it.nchunks; ++i, ++ctr) {
                    // lanes 0-15: output row -> fp16 output tile
                    // lanes 16-31: S <- 2^(G_L) S + kh^T v ; fp16 copy for the next chunk's read-out
                    const uint32_t p = ctr & 1u;
                    group_wait(ctx, &M.os_done[p], (ctr >> 1) & 1u, w, 2, kStateThreads);
                    GLA_EV(14);
                    tc_fence_after();
                    // the exchange slot's chunk total first: its latency hides behind the TMEM read
                    const float b4 = ld_shared_f(smem_u32(&M.b4s[ctr % kSlots][my_c]));
                    const float dec = owner ? ex2(b4) : 0.f;
                    if (owner) gsum += b4;
                    if (!GLA_DBGP(3))
#pragma unroll
                    for (int hb = 0; hb < 2; ++hb) {        // two halves of 32 columns keep the register need bounded
                        float x[32];
                        tmem_row<32>(tmem, quad, kTmOS + 64u * p + 32u * hb, x);
#pragma unroll
                        for (int v = 0; v < 32; ++v)        // lanes 0-15: dec = 0, S is the output row
                            S[32 * hb + v] = fmaf(dec, S[32 * hb + v], x[v]);
                    }
                    GLA_EV(52);
                    tc_fence_before();
                    warp_arrive(&M.os_free[p], l);
                    if (!state_only) {
                        const uint32_t j = c2 & 1u;
                        if constexpr (kGated) {
                            // the fp16 copy of the new state goes out first: the next chunk's read-out waits for it
                            if (owner && !GLA_DBGP(3)) store_row_f16<kD / 8>(base + kOffS16, rho, 0, S);
                            fence_proxy_async_smem();
                            if (i + 1 < it.nchunks) warp_arrive(&M.s16_ready, l);
                            // output rows (lanes 0-15): o * rsqrt(mean(o^2) + eps) goes into the output tile in fp16; the
                            // score group multiplies by w * silu(gate) in place and hands the tile to the store warp
                            if (!owner) {
                                float s4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                                for (int v = 0; v < kD; ++v) s4[v & 3] = fmaf(S[v], S[v], s4[v & 3]);
                                const float ss = (s4[0] + s4[1]) + (s4[2] + s4[3]);
                                const float rinv = P.o_mul * rsqrtf(ss * (P.o_mul * P.o_mul) * (1.f / kD) + P.rms_eps);
#pragma unroll
                                for (int v = 0; v < kD; ++v) S[v] *= rinv;
                            }
                            mbar_wait(ctx, &M.o_free[j], ((c2 >> 1) & 1u) ^ 1u);   // tile's previous store has read it
                            if (!owner && !GLA_DBGP(3)) store_row_f16<kD / 8>(base + kOffOut + j * kTileBytes, rho, 0, S);
                            warp_arrive(&M.o_norm[j], l);
                        } else {
                            if (P.o_mul != 1.f) {         // scale not folded into q (zero, negative or not finite)
                                const float mul = owner ? 1.f : P.o_mul;
#pragma unroll
                                for (int v = 0; v < kD; ++v) S[v] *= mul;
                            }
                            // lanes 16-31: fp16 copy of the new state for the next chunk's read-out;
                            // lanes 0-15: output row into an output tile (the store warp sends it out)
                            mbar_wait(ctx, &M.o_free[j], ((c2 >> 1) & 1u) ^ 1u);   // tile's previous store has read it
                            if (!GLA_DBGP(3))
                                store_row_f16<kD / 8>(owner ? base + kOffS16 : base + kOffOut + j * kTileBytes, rho, 0, S);
                            fence_proxy_async_smem();
                            __syncwarp();
                            if (l == 0) {
                                if (i + 1 < it.nchunks) mbar_arrive(smem_u32(&M.s16_ready));
                                mbar_arrive(smem_u32(&M.o_ready[j]));
                            }
                        }
                        ++c2;
                        GLA_EV(15);
                    }
                    GLA_EV(16);
                }
                };
                if (!state_only && P.gated) run_chunks(std::true_type{});
                else run_chunks(std::false_type{});

                if (state_only) {
                    if (it.seg == 0) {
                        publish(P.incl + slot * (kD * kD) + my_c * kD, 2u);
                    } else {
                        if (owner) P.agg[slot * kAggStride + kD * kD + my_c] = gsum;
                        publish(P.agg + slot * kAggStride + my_c * kD, 1u);
                    }
                }
            }
            if (it.seg == P.NS - 1 && P.sT != nullptr && owner && real_row) {
                float4* dst = reinterpret_cast<float4*>(P.sT + srow);
#pragma unroll
                for (int x4 = 0; x4 < kD / 4; ++x4)
                    dst[x4] = make_float4(S[4 * x4], S[4 * x4 + 1], S[4 * x4 + 2], S[4 * x4 + 3]);
            }
            __syncthreads();   // the item is drained
        }
        GLA_EV(63);
        GLA_EVG(61);
    } else if (w < kWarpGate) {
        // ==================================================================== score group
        // scores of the output-pass chunks: TMEM -> causal mask -> fp16 tile (takes the place of the raw gate tile
        // of the chunk's stage).  Thread: query row 16*quad + (lane & 15), key columns 32*(lane >> 4) .. +31.
        reg_dealloc<kRegsScore>();
        const int quad = w - kStateWarps, stid = tid - kStateThreads;
        const uint32_t rho = 16 * quad + (l & 15);
        const uint32_t j0 = (l >> 4) * 32u;
        while (true) {
            const int item = next_item();
            if (item >= P.num_items) break;
            const ItemInfo it = decode_item(P, item);
            const int npass = it.state_pass ? 2 : 1;
            for (int pass = 0; pass < npass; ++pass) {
                if (it.state_pass && pass == 0) {
                    ctr += it.nchunks;
                    continue;
                }
                // fused epilogue: position along the scan of this thread's output row in the chunk: u, and for column
                // scans its column cc and row rr inside the column (floor division: u < 0 only for rows before the
                // start of a reversed ragged chunk, which are never written)
                int u = 0, rr = 0, cc = 0;
                if (P.gated) {
                    const int p0 = it.first_chunk * kChunk;
                    u = (P.rev ? (P.T - p0 - kChunk) : p0) + static_cast<int>(rho);
                    if (P.Wc > 1) {
                        cc = u / P.Hc;
                        rr = u - cc * P.Hc;
                        if (rr < 0) { rr += P.Hc; --cc; }
                    }
                }
                // fused epilogue, second half: y = (o * rinv) * w * silu(gate) in place on this thread's half row of
                // output tile (cp & 1), which the state group has filled with the normalised outputs of chunk cp; runs
                // one chunk behind the scores so that it never sits on the chain from one chunk's state to the next
                auto gated_epilogue = [&](uint32_t cp, const uint4* gp) {
                    const uint32_t jb = cp & 1u;
                    mbar_wait(ctx, &M.o_norm[jb], (cp >> 1) & 1u);
                    if (gp != nullptr) {       // rows past the end of the sequence are never sent out
                        const uint4* wp = reinterpret_cast<const uint4*>(P.rms_w + j0);
                        const uint32_t row = base + kOffOut + jb * kTileBytes + rho * 128u;
#pragma unroll
                        for (uint32_t m = 0; m < 4; ++m) {
                            const uint32_t a = row + (((((j0 >> 3) + m) ^ rho) & 7u) << 4);
                            const uint4 o4 = ld_shared_v4(a), g4 = __ldg(gp + m), w4 = __ldg(wp + m);
                            const uint32_t ou[4] = {o4.x, o4.y, o4.z, o4.w}, gu[4] = {g4.x, g4.y, g4.z, g4.w},
                                           wu[4] = {w4.x, w4.y, w4.z, w4.w};
                            uint32_t y[4];
#pragma unroll
                            for (int q2 = 0; q2 < 4; ++q2) {
                                const float2 of = unpack_half2(ou[q2]), gf = unpack_half2(gu[q2]), wf = unpack_half2(wu[q2]);
                                y[q2] = pack_half2(of.x * wf.x * silu_f(gf.x), of.y * wf.y * silu_f(gf.y));
                            }
                            st_shared_v4(a, y[0], y[1], y[2], y[3]);
                        }
                    }
                    fence_proxy_async_smem();
                    warp_arrive(&M.o_ready[jb], l);
                };
                // two instantiations of the chunk loop, as in the state group: the plain operator's loop carries none of
                // the fused epilogue's code
                auto run_scores = [&](auto gated_tag) {
                constexpr bool kGated = decltype(gated_tag)::value;
                const uint4* gp_prev = nullptr;
                for (int i = 0; i < it.nchunks; ++i, ++ctr, ++c2) {
                    const uint32_t s = ctr % kNumStages, b = c2 & 1u;
                    const uint32_t a16 = base + kOffStage + s * kStageBytes + 2 * kTileBytes;
                    // fused epilogue: this thread's half row of the chunk's output gate is asked for now, into L2 (the
                    // score group's register budget has no room to hold it)
                    const uint4* gp = nullptr;
                    if constexpr (kGated) {
                        if (u >= 0 && u < P.T) {
                            // the token read at this row of the chunk follows the same mapping as the TMA boxes
                            const long long tok = (P.Wc > 1) ? static_cast<long long>(rr) * P.Wc + cc : u;
                            gp = reinterpret_cast<const uint4*>(
                                P.gate + it.b * P.gate_sb + tok * P.gate_st + it.h * P.gate_sh + j0);
                            prefetch_l2(gp);
                        }
                        if (!P.rev) {
                            u += kChunk;
                            rr += kChunk;
                            while (rr >= P.Hc) { rr -= P.Hc; ++cc; }
                        } else {
                            u -= kChunk;
                            rr -= kChunk;
                            while (rr < 0) { rr += P.Hc; --cc; }
                        }
                    }
                    group_wait(ctx, &M.a_done[b], (c2 >> 1) & 1u, quad, 3, kScoreThreads);
                    GLA_EV(10);
                    tc_fence_after();
                    if (GLA_DBGP(2)) {
                        warp_arrive(&M.a_free[b], l);
                    } else if (!M.wide[ctr % kSlots]) {
                        float x[32];
                        tmem_row<32>(tmem, quad, kTmA + 32u * b, x);
                        tc_fence_before();
                        warp_arrive(&M.a_free[b], l);
                        mask_and_store_scores<32>(P.rev != 0, a16, rho, j0, x);
                    } else {
                        exact_scores(ctx, base_ptr + (a16 - base), base_ptr + kOffQbar + b * kQkBufBytes, stid, kScoreThreads);
                        warp_arrive(&M.a_free[b], l);
                    }
                    fence_proxy_async_smem();
                    warp_arrive(&M.a16_ready[c2 % kNumStages], l);
                    GLA_EV(11);
                    if constexpr (kGated) {
                        if (i > 0) gated_epilogue(c2 - 1u, gp_prev);
                        gp_prev = gp;
                    }
                }
                if constexpr (kGated) {
                    if (it.nchunks > 0) gated_epilogue(c2 - 1u, gp_prev);
                }
                };
                if (P.gated) run_scores(std::true_type{});
                else run_scores(std::false_type{});
            }
            __syncthreads();
        }
    } else if (w < kWarpProducer) {
        // ==================================================================== gate group
        // Two teams of four warps take the chunks in turn (team = chunk parity), each on its own named barrier and
        // its own exchange rows: a team works on a chunk for two chunk periods, and the two teams' instruction
        // streams fill each other's stalls.
        reg_alloc<kRegsGate>();
        const int gw = w - kWarpGate;
        const int team = gw / kTeamWarps, tw = gw % kTeamWarps;
        const uint32_t bar_id = team ? 4u : 1u;
        while (true) {
            const int item = next_item();
            if (item >= P.num_items) break;
            const ItemInfo it = decode_item(P, item);
            const int npass = it.state_pass ? 2 : 1;
            for (int pass = 0; pass < npass; ++pass) {
                const bool state_only = it.state_pass && pass == 0;
                for (int i = 0; i < it.nchunks; ++i, ++ctr) {
                    const uint32_t b = c2 & 1u, k2 = c2;
                    if (!state_only) ++c2;
                    if (static_cast<int>(ctr & 1u) != team) continue;
                    const uint32_t s = ctr % kNumStages;
                    mbar_wait(ctx, &M.full[s], (ctr / kNumStages) & 1u);
                    // the tf32 buffer is free once the score group is done with its previous use (scores read from
                    // TMEM, or the operands stashed for the exact path read from the buffer itself)
                    const uint32_t qbar = state_only ? 0u : base + kOffQbar + b * kQkBufBytes;
                    GLA_EV(12);
                    if (!GLA_DBGP(0))
                        gate_math(ctx, base + kOffStage + s * kStageBytes, qbar, static_cast<int>(ctr),
                                  chunk_valid((it.first_chunk + i) * kChunk, P.T), tw, l, state_only, &M.a_free[b],
                                  ((k2 >> 1) & 1u) ^ 1u, bar_id);
                    warp_arrive(&M.ops_ready[s], l);
                    GLA_EV(13);
                }
            }
            __syncthreads();
        }
    } else {
        // ==================================================================== service warps
        // These four warps run their loops with all 32 lanes, in warp-uniform control flow, and only the issue of
        // an asynchronous instruction (TMA, tcgen05.mma, commit) is left to one elected lane.  Loop counters,
        // descriptors and coordinates then live in uniform registers, which is what those instructions take; a loop
        // run by a single lane inside a divergent branch pays a move from the vector registers per operand and
        // needs three times as long per MMA.
        reg_dealloc<kRegsService>();
        uint32_t n_s16 = 0;   // single barrier: use count (output-MMA role)
        while (true) {
            const int item = next_item();
            if (item >= P.num_items) break;
            const ItemInfo it = decode_item(P, item);
            const int npass = it.state_pass ? 2 : 1;
            if (w == kWarpProducer) {
                // ------------------------------------------------------------ TMA producer
                for (int pass = 0; pass < npass; ++pass) {
                    const bool state_only = it.state_pass && pass == 0;
                    BoxWalker bw(P, it.first_chunk * kChunk);
                    for (int i = 0; i < it.nchunks; ++i, ++ctr) {
                        const uint32_t s = ctr % kNumStages, n = ctr / kNumStages;
                        mbar_wait(ctx, &M.empty[s], (n & 1u) ^ 1u);
                        GLA_EV(30);
                        if (elect_one()) {
                            const int valid = chunk_valid((it.first_chunk + i) * kChunk, P.T);
                            const int ntens = state_only ? 3 : 4;
                            const uint32_t bar = smem_u32(&M.full[s]);
                            mbar_arrive_expect_tx(bar, static_cast<uint32_t>(valid * 128 * ntens));
                            const uint32_t stage = base + kOffStage + s * kStageBytes;
                            bw.for_each(P, [&](int id, int r, int c, int row) {
                                const uint32_t off = static_cast<uint32_t>(row) * 128u;
                                if (!state_only)
                                    tma_load_5d(stage + 0 * kTileBytes + off, &maps.m[TQ][id], bar, 0, it.h, r, c, it.b);
                                tma_load_5d(stage + 1 * kTileBytes + off, &maps.m[TK][id], bar, 0, it.h, r, c, it.b);
                                tma_load_5d(stage + 2 * kTileBytes + off, &maps.m[TG][id], bar, 0, it.h, r, c, it.b);
                                tma_load_5d(stage + 3 * kTileBytes + off, &maps.m[TV][id], bar, 0, it.h, r, c, it.b);
                            });
                        }
                        __syncwarp();
                        bw.advance(P);
                    }
                }
            } else if (w == kWarpMma) {
                // ------------------------------------------------------------ score MMAs (output pass only)
                constexpr uint32_t idA = umma_idesc(FMT_TF32, 0, 0, 64, 32);
                for (int pass = 0; pass < npass; ++pass) {
                    const bool state_only = it.state_pass && pass == 0;
                    for (int i = 0; i < it.nchunks; ++i, ++ctr) {
                        const uint32_t s = ctr % kNumStages, b = c2 & 1u;
                        // a parity wait only tells apart consecutive phases, so this warp has to observe
                        // every phase of the ring, also those of state-only chunks it has nothing to do for
                        mbar_wait(ctx, &M.ops_ready[s], (ctr / kNumStages) & 1u);
                        if (state_only) continue;
                        mbar_wait(ctx, &M.a_free[b], ((c2 >> 1) & 1u) ^ 1u);   // score group done with this buffer's previous use
                        GLA_EV(20);
                        tc_fence_after();
                        const uint32_t wide = __shfl_sync(0xffffffffu, M.wide[ctr % kSlots], 0);
                        if (elect_one()) {
                            if (!wide && !GLA_DBGP(4)) {
                                const uint64_t dQ = umma_desc_sw128(base + kOffQbar + b * kQkBufBytes);
                                const uint64_t dK = umma_desc_sw128(base + kOffQbar + b * kQkBufBytes + kOffKbarRel);
                                const uint32_t tmA = tmem + kTmA + 32u * b;
#pragma unroll
                                for (uint32_t ks = 0; ks < 8; ++ks) {
                                    const uint32_t o = ((ks >> 2) * kTileBytes + (ks & 3) * 32u) >> 4;
                                    umma_tf32(tmA, dQ + o, dK + o, idA, ks);
                                    umma_tf32(tmA + kLane16, dQ + o, dK + o + ((32 * 128) >> 4), idA, ks);
                                }
                            }
                            umma_commit(smem_u32(&M.a_done[b]));
                        }
                        __syncwarp();
                        GLA_EV(21);
                        ++c2;
                    }
                }
            } else if (w == kWarpMma + 1) {
                // ------------------------------------------------------------ output and state MMAs
                constexpr uint32_t idO = umma_idesc(FMT_F16, 0, 1, 64, 64);
                constexpr uint32_t idS = umma_idesc(FMT_F16, 1, 1, 64, 64);
                const uint32_t tmO = tmem + kTmOS, tmS = tmem + kTmOS + kLane16;
                const uint64_t dS16 = umma_desc_sw128(base + kOffS16, 8192);
                for (int pass = 0; pass < npass; ++pass) {
                    const bool state_only = it.state_pass && pass == 0;
                    for (int i = 0; i < it.nchunks; ++i, ++ctr) {
                        const uint32_t s = ctr % kNumStages;
                        const uint32_t stage = base + kOffStage + s * kStageBytes;
                        const uint64_t dq = umma_desc_sw128(stage), dk = umma_desc_sw128(stage + kTileBytes, 8192),
                                       da16 = umma_desc_sw128(stage + 2 * kTileBytes),
                                       dv = umma_desc_sw128(stage + 3 * kTileBytes, 8192);
                        // The O / state-increment accumulators are double-buffered: everything of this chunk that
                        // does not need the incoming state (A.v and kh^T.v) is issued while the state group still
                        // works on the previous chunk; only the read-out qh.S waits for the state, so the serial
                        // chain from one chunk's state to the next is one short MMA group.
                        const uint32_t p = ctr & 1u;
                        const uint32_t tmOp = tmO + 64u * p, tmSp = tmS + 64u * p;
                        mbar_wait(ctx, &M.full[s], (ctr / kNumStages) & 1u);          // v arrives by TMA
                        mbar_wait(ctx, &M.ops_ready[s], (ctr / kNumStages) & 1u);     // qh, kh written in place
                        mbar_wait(ctx, &M.os_free[p], ((ctr >> 1) & 1u) ^ 1u);        // state group has read this buffer's previous use
                        GLA_EV(22);
                        if (!state_only) mbar_wait(ctx, &M.a16_ready[c2 % kNumStages], (c2 / kNumStages) & 1u);
                        GLA_EV(23);
                        tc_fence_after();
                        if (elect_one() && !GLA_DBGP(5)) {
                            if (!state_only) {
#pragma unroll
                                for (uint32_t ks = 0; ks < 4; ++ks) umma_f16(tmOp, da16 + ks * 2u, dv + ks * 128u, idO, ks);
                            }
#pragma unroll
                            for (uint32_t ks = 0; ks < 4; ++ks) umma_f16(tmSp, dk + ks * 128u, dv + ks * 128u, idS, ks);
                        }
                        __syncwarp();
                        if (!state_only) {
                            mbar_wait(ctx, &M.s16_ready, n_s16++ & 1u);
                            tc_fence_after();
                            ++c2;
                        }
                        if (elect_one()) {
                            if (!state_only && !GLA_DBGP(5)) {
#pragma unroll
                                for (uint32_t ks = 0; ks < 4; ++ks) umma_f16(tmOp, dq + ks * 2u, dS16 + ks * 128u, idO, 1);
                            }
                            umma_commit(smem_u32(&M.os_done[p]));
                            // the same completion hands the stage back to the producer: gate math and the score MMAs
                            // are long done with it, and nothing reads it after these MMAs
                            umma_commit(smem_u32(&M.empty[s]));
                        }
                        __syncwarp();
                        GLA_EV(24);
                    }
                }
            } else {
                // ------------------------------------------------------------ store warp
                // sends finished output tiles out by TMA (two tiles, so the state group's work on one chunk overlaps
                // the store of the previous one)
                for (int pass = 0; pass < npass; ++pass) {
                    if (it.state_pass && pass == 0) continue;
                    BoxWalker bw(P, it.first_chunk * kChunk);
                    for (int i = 0; i < it.nchunks; ++i, ++c2) {
                        const uint32_t j = c2 & 1u;
                        mbar_wait(ctx, &M.o_ready[j], (c2 >> 1) & 1u);
                        if (elect_one()) {
                            const uint32_t tile = base + kOffOut + j * kTileBytes;
                            bw.for_each(P, [&](int id, int r, int c, int row) {
                                tma_store_5d(&maps.m[TO][id], tile + static_cast<uint32_t>(row) * 128u, 0, it.h, r, c, it.b);
                            });
                            tma_store_commit();
                            tma_store_wait_read();
                            mbar_arrive(smem_u32(&M.o_free[j]));
                        }
                        __syncwarp();
                        bw.advance(P);
                    }
                }
            }
            __syncthreads();
        }
        if (w == kWarpMma + 2 && elect_one()) tma_store_wait_all();
    }

    tc_fence_before();
    __syncthreads();
    if (w == kWarpProducer) tmem_dealloc(tmem, kTmemCols);
}

}  // namespace gla
