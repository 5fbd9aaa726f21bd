// Chunkwise gated-linear-attention forward for sm_100a: one persistent kernel.
//
// Work decomposition.  A sequence (one batch b, one head h, T tokens along the scan order)
// is cut into 64-token chunks and the chunks into segments of `cps` chunks.  A work item is
// one (sequence, segment); CTAs take items from an atomic ticket so that an item's
// predecessors are always held by CTAs that already run.  For every segment but the last
// of a sequence the CTA first streams k, g, v only and reduces the segment to an aggregate
// (decay, state increment), publishes it, obtains its incoming state from its predecessors
// by a decoupled look-back, and then streams q, k, g, v once more to produce the outputs (the
// pre-pass walks the segment backwards and its copies carry an evict-last L2 priority, so that
// k, g, v are still in L2 then).  Replaces chunk_compute_S_kernel / chunk_scan_*_kernel /
// chunk_fwd_o_kernel of the reference (engine/gtr/backbone/csrc/gla_chunk.cuh:718-1394).
//
// Per chunk, with G the inclusive within-chunk cumulative log gate, G_L its value at the last
// row and R = G_L / 2 a per-channel reference:
//   X  = G - R                                   one tcgen05.mma: X = L g with a constant matrix L of +-1/2
//                                                (lower triangle +1/2, rest -1/2), exact in fp32
//   qt = q*2^X*sqrt(scale)   kt = k*2^-X*sqrt(scale)     fp16, written over q and k in place
//   A  = tril(qt kt^T)                           tcgen05.mma kind::f16 -> TMEM -> fp16 tile
//   O  = A v + qt St                             St = fp16 copy of the scaled state, one accumulator
//   S' = 2^(G_L-R) (.) (2^R (.) S_in + kt^T v)   kt^T v by tcgen05.mma; the rest in fp32 registers
// The state group carries St for the next chunk directly, St' = ha (.) St + hb (.) kt^T v with per-channel
// factors from the two chunks' references, so the chain from one chunk's state to the next holds no MMA:
// the read-out qt St is issued whenever St is there.
// Operands referenced to the middle of the chunk's decay carry exponents of both signs; fp16 holds them
// while no channel decays by more than 2^(2 kRefLimit) over the chunk.  A chunk beyond that (never with
// GTR's gates; the reference's "strong", "bursts" and -1000 tests do) takes references R_q = 0 for q and
// R_k = G_L for k (all exponents <= 0) and computes its scores A exactly, pair by pair, from fp32 gate sums
// -- the role of the reference's exact_attn_chunk (gla_chunk.cuh:258-311), own code.
// The state-only pre-pass uses X = G - G_L (a second constant matrix), whose exponents are never positive.
//
// Who does what.  Three teams of four warps take the chunks in turn; a team does everything of its chunk that
// is elementwise -- gate factors, score mask, output epilogue -- and elected threads of it issue the chunk's
// MMAs (first warp) and its output TMA store (second warp) between those steps, so a chunk is handed from warp to
// warp only through the tensor core.  While a team waits for an MMA the other two work.  A fourth group carries the state; one
// service warp loads the tiles, another issues the gate-sum MMAs as soon as a chunk's tiles have landed.
//
// Tensor memory (512 columns): per team one 64-column accumulator that holds, one after the other, the scores and
// the outputs of its chunk, and one for the gate sums of its next chunk; two for the state increments.  An M = 64
// accumulator occupies lanes 0-15 of each 32-lane quadrant; it is read with the 16x32bx2 shape, which gives lanes
// 0-15 of a warp the first 32 columns of those rows and lanes 16-31 the other 32, so every lane owns half a row.
//
// Shared memory.  A ring of kNumStages stages of {q, k, g, v} tiles filled by TMA (q and k are
// rewritten in place, the gate tile is reused for the fp16 score tile), two fp16 copies of the
// scaled state, one output tile per team, the two constant matrices and a block of barriers and per-chunk
// exchange vectors.  Rows a sequence does not have (ragged last chunk) are filled with zeros by TMA
// boxes placed out of bounds, so no role special-cases them.
#pragma once

#include <type_traits>

#include "gla_device.cuh"
#ifdef GLA_TRACE
#include "gla_trace.cuh"      // development builds only: in-kernel timeline
#else
#define GLA_EV(id) do { } while (0)
#define GLA_EVV(id, val) do { } while (0)
#define GLA_TRACE_PICK(item) do { } while (0)
#endif

namespace gla {

constexpr int kChunk = 64;
constexpr int kD = 64;                    // V, and the widest K
constexpr int kTileBytes = kChunk * 128;  // one fp16 [64 x 64] tile
constexpr int kStageBytes = 4 * kTileBytes;
#ifndef GLA_STAGES
#define GLA_STAGES 5
#endif
constexpr int kCtasPerSm = 1;               // resident CTAs per SM the launch bounds and the grid size assume
constexpr int kNumStages = GLA_STAGES;
// Five warpgroups of four warps: state group, three chunk teams, service warps.
constexpr int kStateWarps = 4, kTeamWarps = 4, kTeams = 3;
constexpr int kStateThreads = 32 * kStateWarps, kTeamThreads = 32 * kTeamWarps;
constexpr int kThreads = kStateThreads + kTeams * kTeamThreads + 128;
constexpr int kTmemCols = 512;
constexpr uint32_t kTmT = 0;              // per team: scores, then outputs of its chunk (64 columns each)
constexpr uint32_t kTmX = 192;            // per team: gate sums relative to the chunk's reference
constexpr uint32_t kTmInc = 384;          // state increments: two buffers of 64 columns
#ifndef GLA_L2HINT
#define GLA_L2HINT 1
#endif
#ifndef GLA_REVPRE
#define GLA_REVPRE 1
#endif
constexpr bool kL2Hints = GLA_L2HINT != 0;
// The pre-pass walks its segment from the last chunk to the first, so that the output pass, which starts at the first,
// meets the tiles in the reverse of the order they were brought into L2: what a least-recently-used cache still holds
// of the segment is what is asked for next.
constexpr bool kBackwardPrePass = GLA_REVPRE != 0;
constexpr int kSlots = 8;                 // per-chunk exchange slots (reference vector, exact-path flag): outlive the stage
static_assert(kSlots >= kNumStages + 3 && (kSlots & (kSlots - 1)) == 0, "exchange slots must outlive the stage ring");
constexpr float kLog2e = 1.4426950408889634f;
// The common reference of a chunk's operands is half its total decay, per channel: q rows before that point and k rows
// after it carry factors above one, at most 2^(decay / 2).  A chunk whose decay stays within 2 * kRefLimit (log2 units,
// every channel) is handled that way.  The host folds sqrt(scale) / 4 into each of q and k (the factor 16 comes back
// in the output epilogue), so fp16 holds inputs of magnitude up to about 2^(18 - kRefLimit) / sqrt(scale).
constexpr float kRefLimit = 14.f;

// tensor ids inside Maps
enum { TQ = 0, TK = 1, TG = 2, TV = 3, TO = 4, TGATE = 5, kNumTensors = 6 };
constexpr int kNumBoxes = 4;              // box heights 64, 16, 4, 1 rows

struct Maps {
    CUtensorMap m[kNumTensors][kNumBoxes];
};

constexpr int kMaxPlanSegments = 16;

struct Params {
    int B, T, H, NT;
    int K;               // key channels per head, 32 or 64.  A K = 32 head runs as a K = 64 head whose upper 32
                         // channels are zero: the tensor maps of q, k, g give the channel dimension its true extent,
                         // so the TMA loads fill channels 32..63 of every tile with zeros without reading anything,
                         // and state rows 32..63 stay zero
    int Hc, Wc;          // column length / number of columns of the scan (row scans: Hc = T, Wc = 1)
    int rev;             // scan runs from the last token to the first
    int NS, cps;         // segments per sequence, chunks per segment
    // Staggered plan (plan != 0; few sequences): NS = r + 1 segments of unequal length for r CTAs per sequence.  Segment
    // 0 is short, runs its output pass at once (its start state is the call's initial state) and publishes the state
    // after it; segments 1 .. r-1 run a pre-pass meanwhile, which takes as long when they are twice as long; the last
    // segment needs no pre-pass and is taken by whichever CTA is free first -- so only r - 1 of r + 1 segments are read
    // twice, and nobody waits.  seg_start[s] is the first chunk of segment s, seg_start[NS] = NT.
    // Relay plan (plan == 2; more sequences than CTAs): NS equal segments and no pre-pass at all.  Every segment but the
    // last publishes the state after its output pass and its successor starts from that; items are handed out
    // segment-major, so a segment's predecessor was taken a whole round of CTAs earlier and has finished by the time
    // anybody asks for it.  The point is the tail: 384 sequences on 148 CTAs are 3 rounds of whole sequences but 2.7
    // rounds' worth of fifths.
    int plan;
    int seg_start[kMaxPlanSegments + 1];
    int num_items;
    int gated;           // fused RMSNorm * w * silu(gate) epilogue
    // The output scale is folded into the exponents of the gate factors (q_exp = log2(scale), half of it on q and half
    // on k, o_mul = 1) when it is positive and finite; otherwise the epilogue multiplies (q_exp = 0, o_mul = scale).
    float q_exp, q_mul, o_mul;
    float inv_norm;      // 1/gk_normalizer, or 0 when g already is a log gate
    float rms_eps;
    const __half* rms_w;      // [64]
    const __half* gate;       // output gate [B,T,H,64] with element strides gate_sb/st/sh
    long long gate_sb, gate_st, gate_sh;
    const float* s0;
    float* sT;
    uint32_t* ctrl;      // [0] ticket, [1] status
    uint32_t* flags;     // per (sequence, segment): 0 none, 1 aggregate, 2 inclusive state
    float* agg;          // per (sequence, segment): 4096 state increment + 64 log2 decay
    float* incl;         // per (sequence, segment): 4096 state after the segment
    uint32_t wait_limit_us;
#ifdef GLA_TRACE
    unsigned long long* trace;
#endif
};

constexpr int kAggStride = kD * kD + kD;

// shared memory map (bytes from a 1024-aligned base)
constexpr int kOffStage = 0;
constexpr int kOffS16 = kNumStages * kStageBytes;         // two fp16 copies of the scaled state (MMA operand)
constexpr int kOffOut = kOffS16 + 2 * kTileBytes;         // one output tile per team (fp16, swizzled)
constexpr int kOffLmat = kOffOut + kTeams * kTileBytes;   // constant matrices of the gate-sum MMA: output pass, pre-pass
constexpr int kOffMisc = kOffLmat + 2 * kTileBytes;
constexpr int kMiscBytes = 4 * 1024;
constexpr int kSmemBytes = kOffMisc + kMiscBytes + 1024;  // + alignment slack
static_assert(kSmemBytes <= 227 * 1024, "shared memory budget");

struct Misc {
    uint64_t full[kNumStages];
    uint64_t empty[kNumStages];
    // A barrier may run at most one phase ahead of its slowest waiter.  Barriers whose producer can run further
    // ahead are rings indexed like the resource they guard (stage, team, or accumulator / tile pair).
    uint64_t ops_ready[kNumStages], g_ready[kNumStages];
    uint64_t x_done[kTeams], x_free[kTeams], a_done[kTeams], o_done[kTeams];
    // inc_free and s16_ready are waited for by the three teams in turn, each of which comes back to them only every
    // third chunk: as rings of two they could be a whole phase behind a fast team (seen once the state group fell two
    // chunks behind while a chunk's tiles came in late), and a wait that is two phases off passes at once.  Rings of
    // four, indexed by the chunk, leave every waiter at most one phase from its barrier.
    uint64_t inc_done[2], inc_free[4], s16_ready[4], s16_free[2];
    uint32_t tmem_base;
    volatile uint32_t abort;
    int item;
    uint32_t wide[kSlots];
    // per chunk and key channel, log2 units: half the chunk's total decay G_L / 2 (output pass) or G_L itself (pre-pass)
    alignas(16) float vec[kSlots][kD];
};
static_assert(sizeof(Misc) <= kMiscBytes, "misc block too large");

enum { WHERE_MBAR = 1, WHERE_LOOKBACK = 2 };

struct Ctx {
    const Params* p;
    Misc* misc;
    uint8_t* base;       // generic pointer to the 1024-aligned shared-memory base
    uint32_t smem;       // the same as a shared-window address
    uint64_t deadline_span_ns;
};

__device__ __forceinline__ void raise_timeout(const Ctx& c, uint32_t where) {
    c.misc->abort = 1;
    atomicCAS(c.p->ctrl + 1, 0u, where);
}

// Bounded wait.  After a time-out in this CTA every later wait returns at once, so all warps
// keep following the protocol (arrivals, named barriers) and the CTA drains and exits; the
// result is then undefined and the status word says so.
__device__ __forceinline__ void mbar_wait_slow(const Ctx& c, uint32_t b, uint32_t parity) {
    const uint64_t t0 = globaltimer_ns();
    uint32_t n = 0;
    while (true) {
        if (mbar_try_wait(b, parity)) return;
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

// Enumerates the TMA boxes that cover one chunk of the scan: f(box_id, r, c, smem_row) with (r, c) the row inside the
// column and the column where the box starts.  The position can be advanced chunk by chunk without a division.
struct BoxWalker {
    int u_lo;     // scan position of the chunk's first row (may be negative for the ragged chunk of a reversed scan)
    int c, r;     // column and row inside the column of max(u_lo, 0)
    __device__ __forceinline__ BoxWalker(const Params& P, int p0) {
        u_lo = P.rev ? (P.T - p0 - kChunk) : p0;
        const int u0 = max(u_lo, 0);
        c = u0 / P.Hc;
        r = u0 - c * P.Hc;
    }
    // boxes over the rows the sequence has
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
    // boxes over the rows of the tile the sequence does not have (loads only): placed out of bounds, the copy
    // engine fills them with zeros.  f(box_id, smem_row)
    template <class F>
    __device__ __forceinline__ void for_each_missing(const Params& P, F f) const {
        int row = u_lo < 0 ? 0 : min(u_lo + kChunk, P.T) - u_lo;        // first missing tile row
        int len = u_lo < 0 ? -u_lo : kChunk - row;
        while (len > 0) {
            const int id = len >= 16 ? 1 : len >= 4 ? 2 : 3;
            const int R = 64 >> (2 * id);
            f(id, row);
            row += R;
            len -= R;
        }
    }
    // one chunk back along the scan
    __device__ __forceinline__ void retreat(const Params& P) {
        if (!P.rev) {
            u_lo -= kChunk;
            r -= kChunk;
            while (r < 0) { r += P.Hc; --c; }
        } else if (u_lo < 0) {
            *this = BoxWalker(P, P.T - u_lo - 2 * kChunk);
        } else {
            u_lo += kChunk;
            r += kChunk;
            while (r >= P.Hc) { r -= P.Hc; ++c; }
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

__device__ __forceinline__ void unpack8(uint4 r, float* x) {
    const float2 a = unpack_half2(r.x), b = unpack_half2(r.y), c = unpack_half2(r.z), d = unpack_half2(r.w);
    x[0] = a.x; x[1] = a.y; x[2] = b.x; x[3] = b.y; x[4] = c.x; x[5] = c.y; x[6] = d.x; x[7] = d.y;
}
__device__ __forceinline__ uint32_t sw_f16(uint32_t row, uint32_t col) {     // col in fp16 elements
    return row * 128u + ((((col >> 3) ^ row) & 7u) << 4) + ((col & 7u) << 1);
}
// address of 16-byte unit `unit` of row `row` in a swizzled tile
__device__ __forceinline__ uint32_t sw_unit(uint32_t tile, uint32_t row, uint32_t unit) {
    return tile + row * 128u + (((unit ^ row) & 7u) << 4);
}
__device__ __forceinline__ uint32_t hmul2_u32(uint32_t a, uint32_t b) {
    __half2 r = __hmul2(*reinterpret_cast<__half2*>(&a), *reinterpret_cast<__half2*>(&b));
    return *reinterpret_cast<uint32_t*>(&r);
}

// Half a row (32 fp32 columns) of an M = 64 accumulator: lanes 0-15 of warp `quad` get columns col .. col+31 of rows
// 16 quad + lane, lanes 16-31 get columns col+32 .. col+63 of rows 16 quad + lane - 16.
__device__ __forceinline__ void tmem_half_row(uint32_t tmem_base, int quad, uint32_t col, float* x) {
    const uint32_t addr = tmem_base + (static_cast<uint32_t>(32 * quad) << 16) + col;
    __syncwarp();   // tcgen05.ld is warp-collective
    tmem_ld_16x32bx2(addr, reinterpret_cast<uint32_t*>(x));
    tmem_ld_wait();
}

// Write 8*N8 floats as fp16 into 16-byte units unit0.. of one row of a swizzled tile.
template <int N8>
__device__ __forceinline__ void store_row_f16(uint32_t tile, uint32_t row, uint32_t unit0, const float* x) {
#pragma unroll
    for (uint32_t m = 0; m < N8; ++m)
        st_shared_v4(sw_unit(tile, row, unit0 + m), pack_half2(x[8 * m], x[8 * m + 1]), pack_half2(x[8 * m + 2], x[8 * m + 3]),
                     pack_half2(x[8 * m + 4], x[8 * m + 5]), pack_half2(x[8 * m + 6], x[8 * m + 7]));
}

// ------------------------------------------------------------------------------------------
// The exact path (rare, out of line): a chunk whose decay exceeds what fp16 operands referenced to its middle can
// hold.  Thread (w, l) of the team owns physical row rho = 16 w + (l & 15) and the half hf = l >> 4.
//  * exact scores: A[i][j] = scale * sum_c q[i][c] k[j][c] 2^(G[i][c] - G[j][c]) for the keys j of this thread's key half
//    (physical columns 32 hf .. +31) at or before query i = this row along the scan, from the raw q, k and the log gates of
//    the stage, written as fp32 into the team's accumulator in TMEM (the score step then treats the chunk like any other);
//  * q and k rewritten in place with the references R_q = 0 and R_k = G_L (every exponent <= 0).
// Gate sums are rebuilt from the gate tile with running sums; nothing of this weighs on the common path.
__device__ __noinline__ void gate_wide_chunk(bool rev, float q_exp, float q_mul, uint32_t stage, uint32_t tmem_a, int w, int l,
                                             uint32_t bar_id) {
    const uint32_t tq = stage, tk = stage + kTileBytes, tg = stage + 2 * kTileBytes;
    const uint32_t rho = 16u * w + (l & 15u), hf = static_cast<uint32_t>(l) >> 4;
    const int i = rev ? 63 - static_cast<int>(rho) : static_cast<int>(rho);          // logical query row
    float sres[32];
#pragma unroll
    for (int x = 0; x < 32; ++x) sres[x] = 0.f;
    // two passes over the channel halves keep the registers bounded
#pragma unroll 1
    for (uint32_t ch = 0; ch < 2; ++ch) {
        float qv[32], D[32];
#pragma unroll
        for (uint32_t m = 0; m < 4; ++m) {
            unpack8(ld_shared_v4(sw_unit(tq, rho, 4u * ch + m)), qv + 8 * m);
#pragma unroll
            for (int e = 0; e < 8; ++e) D[8 * m + e] = 0.f;
        }
        // walk the keys from the query backwards along the scan: D = G[i] - G[j]
#pragma unroll 1
        for (int j = i; j >= 0; --j) {
            const uint32_t pj = rev ? 63u - j : static_cast<uint32_t>(j);            // physical key row / column
            if ((pj >> 5) == hf) {
                float s = 0.f;
#pragma unroll
                for (uint32_t m = 0; m < 4; ++m) {
                    float kv[8];
                    unpack8(ld_shared_v4(sw_unit(tk, pj, 4u * ch + m)), kv);
#pragma unroll
                    for (int e = 0; e < 8; ++e) s = fmaf(qv[8 * m + e] * kv[e], ex2(D[8 * m + e]), s);
                }
                sres[pj & 31u] += s;
            }
            // next key is one step earlier: its gap to the query grows by this key's own gate
#pragma unroll
            for (uint32_t m = 0; m < 4; ++m) {
                float gv[8];
                unpack8(ld_shared_v4(sw_unit(tg, pj, 4u * ch + m)), gv);
#pragma unroll
                for (int e = 0; e < 8; ++e) D[8 * m + e] = fmaf(gv[e], kLog2e, D[8 * m + e]);
            }
        }
    }
#pragma unroll
    for (int x = 0; x < 32; ++x) sres[x] *= q_mul;
    __syncwarp();
    tmem_st_16x32bx2(tmem_a + (static_cast<uint32_t>(32 * w) << 16), reinterpret_cast<const uint32_t*>(sres));
    tmem_st_wait();
    tc_fence_before();
    named_bar_sync(bar_id, kTeamThreads);                 // every thread has read the raw rows it needs
    // this row's gate sums G (inclusive) and the chunk totals G_L, channels 32 hf .. +31
    float G[32], GL[32];
#pragma unroll
    for (int x = 0; x < 32; ++x) G[x] = GL[x] = 0.f;
#pragma unroll 1
    for (int t = 0; t < 64; ++t) {
        const uint32_t pt = rev ? 63u - t : static_cast<uint32_t>(t);
#pragma unroll
        for (uint32_t m = 0; m < 4; ++m) {
            float gv[8];
            unpack8(ld_shared_v4(sw_unit(tg, pt, 4u * hf + m)), gv);
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                GL[8 * m + e] = fmaf(gv[e], kLog2e, GL[8 * m + e]);
                if (t <= i) G[8 * m + e] = fmaf(gv[e], kLog2e, G[8 * m + e]);
            }
        }
    }
    const float hk = 0.5f * q_exp, hq = q_exp - hk;
#pragma unroll
    for (uint32_t m = 0; m < 4; ++m) {
        float qv[8], kv[8];
        const uint32_t aq = sw_unit(tq, rho, 4u * hf + m), ak = sw_unit(tk, rho, 4u * hf + m);
        unpack8(ld_shared_v4(aq), qv);
        unpack8(ld_shared_v4(ak), kv);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            qv[e] *= ex2(G[8 * m + e] + hq);
            kv[e] *= ex2(GL[8 * m + e] - G[8 * m + e] + hk);
        }
        st_shared_v4(aq, pack_half2_sat(qv[0], qv[1]), pack_half2_sat(qv[2], qv[3]), pack_half2_sat(qv[4], qv[5]),
                     pack_half2_sat(qv[6], qv[7]));
        st_shared_v4(ak, pack_half2_sat(kv[0], kv[1]), pack_half2_sat(kv[2], kv[3]), pack_half2_sat(kv[4], kv[5]),
                     pack_half2_sat(kv[6], kv[7]));
    }
}

// Raw-logit gates (gk_normalizer > 0): the gate tile is rewritten in place as fp16 log gates, logsigmoid(x) / normalizer,
// before the gate-sum MMA reads it; rows the sequence does not have (zero-filled) must not decay.
__device__ __noinline__ void logits_to_log_gates(uint32_t tg, float inv_norm, bool rev, int valid, int w, int l) {
    const uint32_t rho = 16u * w + (l & 15u), hf = static_cast<uint32_t>(l) >> 4;
    const int t = rev ? 63 - static_cast<int>(rho) : static_cast<int>(rho);
#pragma unroll
    for (uint32_t m = 0; m < 4; ++m) {
        const uint32_t a = sw_unit(tg, rho, 4u * hf + m);
        float gv[8];
        unpack8(ld_shared_v4(a), gv);
        uint32_t h[4];
#pragma unroll
        for (int e = 0; e < 4; ++e)
            h[e] = t < valid ? pack_half2_sat(logsigmoid_f(gv[2 * e]) * inv_norm, logsigmoid_f(gv[2 * e + 1]) * inv_norm) : 0u;
        st_shared_v4(a, h[0], h[1], h[2], h[3]);
    }
    fence_proxy_async_smem();
}

// Causal mask along the scan on the 32 score columns j0.. of query row rho (keep key j0 + j at or before the query;
// at or after it for reversed scans), then the fp16 tile.  Branch-free selects: the two half-warps sit on different
// sides of the diagonal.
__device__ __forceinline__ void mask_and_store_scores(bool rev, uint32_t a16, uint32_t rho, uint32_t j0, float* x) {
    const int lim = static_cast<int>(rho) - static_cast<int>(j0);
#pragma unroll
    for (int j = 0; j < 32; ++j) x[j] = (rev ? (j >= lim) : (j <= lim)) ? x[j] : 0.f;
    store_row_f16<4>(a16, rho, j0 >> 3, x);
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
    int publish_end;     // the state after the segment's output pass is what its successors start from
};

__device__ __forceinline__ ItemInfo decode_item(const Params& P, int item) {
    ItemInfo it;
    const int nseq = P.B * P.H;
    it.seg = item / nseq;
    it.seq = item - it.seg * nseq;
    it.b = it.seq / P.H;
    it.h = it.seq - it.b * P.H;
    if (P.plan == 2) {
        it.first_chunk = it.seg * P.cps;
        it.nchunks = min(P.cps, P.NT - it.first_chunk);
        it.state_pass = 0;
        it.publish_end = (it.seg < P.NS - 1) ? 1 : 0;
    } else if (P.plan) {
        it.first_chunk = P.seg_start[it.seg];
        it.nchunks = P.seg_start[it.seg + 1] - it.first_chunk;
        it.state_pass = (it.seg > 0 && it.seg < P.NS - 1) ? 1 : 0;
        it.publish_end = (it.seg == 0 && P.NS > 1) ? 1 : 0;
    } else {
        it.first_chunk = it.seg * P.cps;
        it.nchunks = min(P.cps, P.NT - it.first_chunk);
        it.state_pass = (it.seg < P.NS - 1) ? 1 : 0;
        it.publish_end = 0;
    }
    return it;
}

// Warp roles (one CTA per SM, 20 warps in five warpgroups).  Warp w of a group that reads tensor memory works on the
// rows of quadrant w % 4: lanes 0-15 on the first 32 columns of rows 16 (w % 4) + lane, lanes 16-31 on the other 32.
//   warps 0..3    state group   reads the state increments kt^T v from TMEM and carries the (scaled) state in fp32
//                               registers, half a row per thread; writes its fp16 copy for the next chunk's read-out
//                               MMA; look-back and publication of segment states
//   warps 4..15   three teams   chunk n belongs to team n % 3.  Per chunk: gate sums from TMEM -> qt, kt in place ->
//                               [MMAs: scores, state increment] -> scores from TMEM -> mask -> fp16 tile -> [MMAs: A v,
//                               qt St] -> outputs from TMEM -> (RMSNorm * w * silu(gate)) -> fp16 tile -> [TMA store].
//                               The steps in brackets are issued by one elected thread of the team's first warp.
//   warp 16       TMA producer
//   warp 17       gate-sum MMAs L g, issued as soon as a chunk's tiles have landed and its team's buffer is free
//   warps 18, 19  idle
// The chain from one chunk's state to the next runs inside the state group alone (an fp32 multiply-add per element
// on the increment read from TMEM).  Each warpgroup sets its own register budget (setmaxnreg): the budgets re-divide
// what the CTA got at launch (kThreads x 96 registers) and must not add up to more than that, because an increase
// waits, without limit, until the other groups have released enough.
#ifndef GLA_REGS_STATE
#define GLA_REGS_STATE 96
#define GLA_REGS_TEAM 112
#define GLA_REGS_SERVICE 40
#endif
constexpr int kRegsState = GLA_REGS_STATE, kRegsTeam = GLA_REGS_TEAM, kRegsService = GLA_REGS_SERVICE;
constexpr int kLaunchRegs = 96;
constexpr int kRegBudgetTotal = kStateThreads * kRegsState + kTeams * kTeamThreads * kRegsTeam + 128 * kRegsService;
static_assert(kRegBudgetTotal <= kThreads * kLaunchRegs, "register budgets exceed what the CTA is launched with");
template <int N> __device__ __forceinline__ void reg_budget() {
    if constexpr (N > kLaunchRegs) reg_alloc<N>();
    else if constexpr (N < kLaunchRegs) reg_dealloc<N>();
}

// One instantiation per combination of fused epilogue, raw-logit gates and scan sense: each holds only the code of its
// own case, which keeps the instruction working set of the concurrently running roles small.
template <bool kGated, bool kLogits, bool kRev>
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
    int trace_slot = -2;
    const long long trace_t0 = clock64();
#endif
    GLA_EV(1);
    GLA_EVV(2, globaltimer_ns());
    constexpr int kWarpTeam = kStateWarps;
    constexpr int kWarpProducer = kWarpTeam + kTeams * kTeamWarps, kWarpX = kWarpProducer + 1;

    Ctx ctx;
    ctx.p = &P;
    ctx.misc = &M;
    ctx.base = base_ptr;
    ctx.smem = base;
    ctx.deadline_span_ns = static_cast<uint64_t>(P.wait_limit_us) * 1000ull;

    if (tid == 0) {
        for (int s = 0; s < kNumStages; ++s) {
            mbar_init(smem_u32(&M.full[s]), 1);
            mbar_init(smem_u32(&M.empty[s]), 1);
            mbar_init(smem_u32(&M.ops_ready[s]), 1);
            mbar_init(smem_u32(&M.g_ready[s]), kTeamWarps);
        }
        for (int t = 0; t < kTeams; ++t) {
            mbar_init(smem_u32(&M.x_done[t]), 1);
            mbar_init(smem_u32(&M.x_free[t]), kTeamWarps);
            mbar_init(smem_u32(&M.a_done[t]), 1);
            mbar_init(smem_u32(&M.o_done[t]), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(smem_u32(&M.inc_done[b]), 1);
            mbar_init(smem_u32(&M.s16_free[b]), 1);
        }
        for (int b = 0; b < 4; ++b) {
            mbar_init(smem_u32(&M.inc_free[b]), kStateWarps);
            mbar_init(smem_u32(&M.s16_ready[b]), kStateWarps);
        }
        M.abort = 0;
        fence_mbar_init();
    }
    // The constant matrices of the gate-sum MMA, as K-major operands (row = output row, 128 B = the 64 source rows), in
    // physical row order: for a reversed scan the rows along the scan run from 63 down to 0.
    //   output pass: +1/2 where the source row is at or before the output row along the scan, -1/2 elsewhere  (G - G_L/2)
    //   pre-pass:    -1 where the source row is after the output row, 0 elsewhere                            (G - G_L)
    for (int e = tid; e < kChunk * kChunk; e += kThreads) {
        const uint32_t r = static_cast<uint32_t>(e) >> 6, s = static_cast<uint32_t>(e) & 63u;
        const bool at_or_before = kRev ? (s >= r) : (s <= r);
        const uint32_t o = sw_f16(r, s);
        *reinterpret_cast<__half*>(base_ptr + kOffLmat + o) = __float2half(at_or_before ? 0.5f : -0.5f);
        *reinterpret_cast<__half*>(base_ptr + kOffLmat + kTileBytes + o) = __float2half(at_or_before ? 0.f : -1.f);
    }
    fence_proxy_async_smem();
    if (w == kWarpProducer) {
        tmem_alloc(smem_u32(&M.tmem_base), kTmemCols);
        tmem_relinquish();
    }
    if (w == kWarpX && l == 0) {
        for (int t = 0; t < TGATE; ++t) tma_prefetch_desc(&maps.m[t][0]);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    GLA_EV(5);
    const uint32_t tmem = __shfl_sync(0xffffffffu, M.tmem_base, 0);
    constexpr bool logits = kLogits;
    constexpr bool rev = kRev;
    const float hk = 0.5f * P.q_exp, hq = P.q_exp - hk;       // k's and q's share of the output scale (log2)

    // Every role walks the same sequence of work items and chunks and keeps its own counters:
    //   ctr  chunks seen so far (both passes): stage = ctr % kNumStages, exchange slot = ctr % kSlots,
    //        increment accumulator = ctr & 1, team = ctr % kTeams (its use count of the team's buffers = ctr / kTeams)
    //   c2   output-pass chunks seen so far: state copy = c2 & 1
    // A barrier of a ring of R entries used for the u-th time is waited for with parity (u / R) & 1; "the entry is free
    // for its u-th use" is the completion of the release of use u - R, parity ((u / R) & 1) ^ 1 (true at once for u < R).
    uint32_t ctr = 0, c2 = 0;
    // Work items come from a ticket counter; all roles fetch the same item at the same two block barriers.
    auto next_item = [&]() -> int {
        if (tid == 0) M.item = static_cast<int>(atomicAdd(P.ctrl, 1u));
        __syncthreads();
        GLA_TRACE_PICK(M.item);
        GLA_EVV(9, trace_t0);
        GLA_EV(3);
        GLA_EVV(6, M.item);
        return __shfl_sync(0xffffffffu, M.item, 0);   // known to be warp-uniform
    };

    if (w < kStateWarps) {
        // ==================================================================== state group
        reg_budget<kRegsState>();
        const int quad = w;
        const uint32_t hf = static_cast<uint32_t>(l) >> 4;
        const int my_c = 16 * quad + (l & 15);          // state row (key channel); this thread holds its columns 32 hf .. +31
        const uint32_t rho = static_cast<uint32_t>(my_c);
        float S[32];                                    // scaled by 2^(reference of the chunk that reads it next)
        // per-channel log2 factors of a chunk from its exchange slot: rq (reference of the state copy its read-out uses),
        // ta = G_L - rq, tb = G_L - R_k - hk, gl = G_L
        auto slot_rq = [&](uint32_t n) -> float {
            const float v = ld_shared_f(smem_u32(&M.vec[n & (kSlots - 1)][my_c]));
            return M.wide[n & (kSlots - 1)] ? hk : v + hk;
        };
        while (true) {
            const int item = next_item();
            if (item >= P.num_items) break;
            const ItemInfo it = decode_item(P, item);
            const int npass = it.state_pass ? 2 : 1;
            const size_t srow = (static_cast<size_t>(it.seq) * P.K + my_c) * kD + 32 * hf;   // this thread's half row of the state
            const bool real_row = my_c < P.K;      // rows of channels a K = 32 head does not have are zero throughout
            const size_t slot = static_cast<size_t>(it.seq) * P.NS + it.seg;
            const size_t hoff = static_cast<size_t>(my_c) * kD + 32 * hf;                    // the same inside one 64 x 64 state
            float gsum = 0.f;       // log2 of the segment's total decay for channel my_c

            auto load_initial = [&]() {
#pragma unroll
                for (int x = 0; x < 32; ++x) S[x] = 0.f;
                if (real_row && P.s0 != nullptr) {
                    const float4* src = reinterpret_cast<const float4*>(P.s0 + srow);
#pragma unroll
                    for (int x = 0; x < 8; ++x) {
                        const float4 v4 = __ldg(src + x);
                        S[4 * x] = v4.x; S[4 * x + 1] = v4.y; S[4 * x + 2] = v4.z; S[4 * x + 3] = v4.w;
                    }
                }
            };
            auto publish = [&](float* dst_half_row, uint32_t flag_value) {
                float4* dst = reinterpret_cast<float4*>(dst_half_row);
#pragma unroll
                for (int x4 = 0; x4 < 8; ++x4)
                    dst[x4] = make_float4(S[4 * x4], S[4 * x4 + 1], S[4 * x4 + 2], S[4 * x4 + 3]);
                // The group barrier orders every thread's stores before thread 0's release store, and a release is
                // cumulative over what its thread has synchronised with: no per-thread fence is needed.
                named_bar_sync(2, kStateThreads);
                if (tid == 0) st_release_gpu(P.flags + slot, flag_value);
            };

            for (int pass = 0; pass < npass; ++pass) {
                const bool state_only = it.state_pass && pass == 0;
                const bool back = state_only && kBackwardPrePass;
                if (state_only || it.seg == 0) {
                    // the pre-pass reduces the segment to (decay, increment) from a zero state; segment 0 starts
                    // from the initial state in either pass (a backward pre-pass adds it at the end)
                    if (it.seg == 0 && !back) load_initial();
                    else {
#pragma unroll
                        for (int x = 0; x < 32; ++x) S[x] = 0.f;
                    }
                } else {
                    // decoupled look-back: S <- state entering this segment
                    GLA_EV(60);
#pragma unroll
                    for (int x = 0; x < 32; ++x) S[x] = 0.f;
                    float dlog = 0.f;
                    int j = it.seg - 1;
                    const uint64_t t0 = globaltimer_ns();
                    while (true) {
                        const size_t sj = static_cast<size_t>(it.seq) * P.NS + j;
                        // one lane per warp polls (the CTAs of later segments wait here for a whole pre-pass of
                        // their predecessors), the warp barrier of the shuffle passes the acquired view on
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
                        const float4* src = reinterpret_cast<const float4*>(
                            (inclusive ? P.incl + sj * (kD * kD) : P.agg + sj * kAggStride) + hoff);
#pragma unroll
                        for (int x4 = 0; x4 < 8; ++x4) {
                            const float4 v4 = __ldcg(src + x4);
                            S[4 * x4] = fmaf(dacc, v4.x, S[4 * x4]);
                            S[4 * x4 + 1] = fmaf(dacc, v4.y, S[4 * x4 + 1]);
                            S[4 * x4 + 2] = fmaf(dacc, v4.z, S[4 * x4 + 2]);
                            S[4 * x4 + 3] = fmaf(dacc, v4.w, S[4 * x4 + 3]);
                        }
                        if (!inclusive) dlog += __ldcg(P.agg + sj * kAggStride + kD * kD + my_c);
                        if (inclusive) break;
                        --j;   // never drops below 0: segment 0 only ever publishes an inclusive state
                        if (j < 0) break;
                    }
                    if (it.state_pass) {
                        // inclusive state after this segment = decay * incoming + increment
                        const float dseg = ex2(gsum);
                        const float4* inc = reinterpret_cast<const float4*>(P.agg + slot * kAggStride + hoff);
                        float4* dst = reinterpret_cast<float4*>(P.incl + slot * (kD * kD) + hoff);
#pragma unroll
                        for (int x4 = 0; x4 < 8; ++x4) {
                            const float4 a4 = __ldcg(inc + x4);
                            dst[x4] = make_float4(fmaf(dseg, S[4 * x4], a4.x), fmaf(dseg, S[4 * x4 + 1], a4.y),
                                                  fmaf(dseg, S[4 * x4 + 2], a4.z), fmaf(dseg, S[4 * x4 + 3], a4.w));
                        }
                        named_bar_sync(2, kStateThreads);
                        if (tid == 0) st_release_gpu(P.flags + slot, 2u);
                    }
                }
                GLA_EV(61);
                if (it.nchunks > 0) {
                    // the first chunk's reference is known once its gate math is done; every chunk's `ops_ready` phase
                    // is waited for exactly once by this group (here, or as "the next chunk" inside the loop)
                    mbar_wait(ctx, &M.ops_ready[ctr % kNumStages], (ctr / kNumStages) & 1u);
                    if (!state_only) {
                        const float f0 = ex2(slot_rq(ctr));
#pragma unroll
                        for (int x = 0; x < 32; ++x) S[x] *= f0;
                        const uint32_t j = c2 & 1u;
                        mbar_wait(ctx, &M.s16_free[j], ((c2 >> 1) & 1u) ^ 1u);
                        store_row_f16<4>(base + kOffS16 + j * kTileBytes, rho, 4u * hf, S);
                        fence_proxy_async_smem();
                        warp_arrive(&M.s16_ready[c2 & 3u], l);
                    }
                }
                for (int i = 0; i < it.nchunks; ++i, ++ctr) {
                    const uint32_t p = ctr & 1u;
                    const bool has_next = i + 1 < it.nchunks;
                    // factors of this step: S' = ha * S + hb * (kt^T v), referenced to the next chunk's R_q
                    float rq_next = 0.f;
                    if (has_next) {
                        const uint32_t cn = ctr + 1;
                        mbar_wait(ctx, &M.ops_ready[cn % kNumStages], (cn / kNumStages) & 1u);
                        if (!state_only) rq_next = slot_rq(cn);
                    }
                    const float v = ld_shared_f(smem_u32(&M.vec[ctr & (kSlots - 1)][my_c]));
                    float ta, tb;
                    if (state_only) {
                        // forward: S' = 2^G_L S + inc; backward: S' = S + 2^(decay of the chunks after this one) inc
                        ta = back ? 0.f : v;
                        tb = back ? gsum : 0.f;
                        gsum += v;
                    }
                    else {
                        const bool wide = M.wide[ctr & (kSlots - 1)] != 0u;
                        ta = wide ? 2.f * v - hk : v - hk;
                        tb = wide ? -hk : v - hk;
                        gsum += 2.f * v;
                    }
                    const float ha = ex2(rq_next + ta), hb = ex2(rq_next + tb);
                    GLA_EV(50);
                    group_wait(ctx, &M.inc_done[p], (ctr >> 1) & 1u, w, 2, kStateThreads);
                    GLA_EV(14);
                    tc_fence_after();
                    {
                        float x[32];
                        tmem_half_row(tmem, quad, kTmInc + 64u * p, x);
#pragma unroll
                        for (int e = 0; e < 32; ++e) S[e] = fmaf(ha, S[e], hb * x[e]);
                    }
                    GLA_EV(51);
                    tc_fence_before();
                    warp_arrive(&M.inc_free[ctr & 3u], l);
                    if (!state_only) {
                        if (has_next) {
                            const uint32_t cn2 = c2 + 1, j = cn2 & 1u;
                            mbar_wait(ctx, &M.s16_free[j], ((cn2 >> 1) & 1u) ^ 1u);
                            store_row_f16<4>(base + kOffS16 + j * kTileBytes, rho, 4u * hf, S);
                            fence_proxy_async_smem();
                            warp_arrive(&M.s16_ready[cn2 & 3u], l);
                        }
                        ++c2;
                    }
                    GLA_EV(15);
                }

                GLA_EV(62);
                if (state_only) {
                    if (back && it.seg == 0 && real_row && P.s0 != nullptr) {
                        const float dtot = ex2(gsum);
                        const float4* src = reinterpret_cast<const float4*>(P.s0 + srow);
#pragma unroll
                        for (int x = 0; x < 8; ++x) {
                            const float4 v4 = __ldg(src + x);
                            S[4 * x] = fmaf(dtot, v4.x, S[4 * x]); S[4 * x + 1] = fmaf(dtot, v4.y, S[4 * x + 1]);
                            S[4 * x + 2] = fmaf(dtot, v4.z, S[4 * x + 2]); S[4 * x + 3] = fmaf(dtot, v4.w, S[4 * x + 3]);
                        }
                    }
                    if (it.seg == 0) {
                        publish(P.incl + slot * (kD * kD) + hoff, 2u);
                    } else {
                        if (hf == 0) P.agg[slot * kAggStride + kD * kD + my_c] = gsum;
                        publish(P.agg + slot * kAggStride + hoff, 1u);
                    }
                }
            }
            if (it.publish_end) publish(P.incl + slot * (kD * kD) + hoff, 2u);
            if (it.seg == P.NS - 1 && P.sT != nullptr && real_row) {
                float4* dst = reinterpret_cast<float4*>(P.sT + srow);
#pragma unroll
                for (int x4 = 0; x4 < 8; ++x4)
                    dst[x4] = make_float4(S[4 * x4], S[4 * x4 + 1], S[4 * x4 + 2], S[4 * x4 + 3]);
            }
            __syncthreads();   // the item is drained
        }
    } else if (w < kWarpProducer) {
        // ==================================================================== chunk teams
        // Thread (tw, l): row rho = 16 tw + (l & 15) of the chunk (physical order), columns 32 (l >> 4) .. +31 of whatever
        // the step works on: key channels (gate math), key rows (scores), value channels (outputs).
        reg_budget<kRegsTeam>();
        const int team = (w - kWarpTeam) / kTeamWarps, tw = (w - kWarpTeam) % kTeamWarps;
        const uint32_t bar_id = 3u + static_cast<uint32_t>(team);
        const uint32_t rho = 16u * tw + (l & 15u), hf = static_cast<uint32_t>(l) >> 4, j0 = 32u * hf;
        const uint32_t tmT = tmem + kTmT + 64u * team, tmXt = kTmX + 64u * team;
        const uint32_t out_tile = base + kOffOut + team * kTileBytes;
        constexpr uint32_t idA = umma_idesc(FMT_F16, 0, 0, 64, 64);     // qt x kt^T
        constexpr uint32_t idS = umma_idesc(FMT_F16, 1, 1, 64, 64);     // kt^T x v
        constexpr uint32_t idO = umma_idesc(FMT_F16, 0, 1, 64, 64);     // A16 x v, qt x St
        const bool issuer = tw == 0;                  // the team's first warp issues its MMAs (one elected lane),
        const bool storer = tw == 1;                  // its second warp the output stores
        const uint64_t pol_stream = l2_policy_stream();
        uint32_t oturn = 0;                           // output-pass chunks this team has taken: use count of a_done / o_done
        while (true) {
            const int item = next_item();
            if (item >= P.num_items) break;
            const ItemInfo it = decode_item(P, item);
            const int npass = it.state_pass ? 2 : 1;
            for (int pass = 0; pass < npass; ++pass) {
                const bool state_only = it.state_pass && pass == 0;
                for (int i = 0; i < it.nchunks; ++i, ++ctr) {
                    const uint32_t k2 = c2;
                    if (!state_only) ++c2;
                    if (ctr % kTeams != static_cast<uint32_t>(team)) continue;
                    const uint32_t s = ctr % kNumStages, turn = ctr / kTeams, p = ctr & 1u, slot = ctr & (kSlots - 1);
                    const uint32_t stage = base + kOffStage + s * kStageBytes;
                    const uint32_t tq = stage, tk = stage + kTileBytes, tg = stage + 2 * kTileBytes;
                    mbar_wait(ctx, &M.full[s], (ctr / kNumStages) & 1u);
                    GLA_EV(12);
                    if (logits) {
                        const int ci = it.first_chunk + ((state_only && kBackwardPrePass) ? it.nchunks - 1 - i : i);
                        logits_to_log_gates(tg, P.inv_norm, rev, chunk_valid(ci * kChunk, P.T), tw, l);
                        warp_arrive(&M.g_ready[s], l);
                    }
                    // ---- gate sums of this thread's row and channel half
                    float x[32];
                    mbar_wait(ctx, &M.x_done[team], turn & 1u);
                    tc_fence_after();
                    tmem_half_row(tmem, tw, tmXt, x);
                    tc_fence_before();
                    warp_arrive(&M.x_free[team], l);
                    GLA_EV(40);
                    if (state_only) {
                        // x = G - G_L >= 0 (natural log units); kt = k 2^-x, every factor <= 1.  The first row along the scan sees
                        // G_L = g_first - x and leaves it for the state group.
                        if (rho == (rev ? 63u : 0u)) {
#pragma unroll
                            for (uint32_t m = 0; m < 4; ++m) {
                                float gv[8];
                                unpack8(ld_shared_v4(sw_unit(tg, rho, 4u * hf + m)), gv);
                                const uint32_t o = smem_u32(&M.vec[slot][32u * hf + 8u * m]);
                                st_shared_f4(o, (gv[0] - x[8 * m]) * kLog2e, (gv[1] - x[8 * m + 1]) * kLog2e,
                                             (gv[2] - x[8 * m + 2]) * kLog2e, (gv[3] - x[8 * m + 3]) * kLog2e);
                                st_shared_f4(o + 16, (gv[4] - x[8 * m + 4]) * kLog2e, (gv[5] - x[8 * m + 5]) * kLog2e,
                                             (gv[6] - x[8 * m + 6]) * kLog2e, (gv[7] - x[8 * m + 7]) * kLog2e);
                            }
                        }
#pragma unroll
                        for (uint32_t m = 0; m < 4; ++m) {
                            const uint32_t ak = sw_unit(tk, rho, 4u * hf + m);
                            const uint4 kr = ld_shared_v4(ak);
                            uint32_t f[4];
#pragma unroll
                            for (int e = 0; e < 4; ++e)
                                f[e] = pack_half2(ex2(-kLog2e * x[8 * m + 2 * e]), ex2(-kLog2e * x[8 * m + 2 * e + 1]));
                            st_shared_v4(ak, hmul2_u32(kr.x, f[0]), hmul2_u32(kr.y, f[1]), hmul2_u32(kr.z, f[2]), hmul2_u32(kr.w, f[3]));
                        }
                        fence_proxy_async_smem();
                        named_bar_sync(bar_id, kTeamThreads);
                        if (issuer) {
                            if (ctr >= 2u) mbar_wait(ctx, &M.inc_free[(ctr - 2u) & 3u], ((ctr - 2u) >> 2) & 1u);    // state group has read this buffer's previous use
                            tc_fence_after();
                            if (elect_one()) {
                                const uint64_t dk = umma_desc_sw128(tk, 8192), dv = umma_desc_sw128(stage + 3 * kTileBytes, 8192);
                                const uint32_t tmI = tmem + kTmInc + 64u * p;
#pragma unroll
                                for (uint32_t ks = 0; ks < 4; ++ks) umma_f16(tmI, dk + ks * 128u, dv + ks * 128u, idS, ks);
                                umma_commit(smem_u32(&M.inc_done[p]));
                                umma_commit(smem_u32(&M.empty[s]));
                                mbar_arrive(smem_u32(&M.ops_ready[s]));
                            }
                            __syncwarp();
                        }
                        GLA_EV(13);
                        continue;
                    }
                    // ---- output pass.  x = G - G_L / 2 (natural log units): qt = q 2^(x + hq), kt = k 2^(-x + hk)
                    if (tw == (rev ? 0 : 3)) {              // the warp that holds the last row along the scan
                        const bool last = rho == (rev ? 0u : 63u);
                        bool far = false;
                        if (last) {
#pragma unroll
                            for (uint32_t m = 0; m < 8; ++m) {
                                const float h0 = x[4 * m] * kLog2e, h1 = x[4 * m + 1] * kLog2e, h2 = x[4 * m + 2] * kLog2e,
                                            h3 = x[4 * m + 3] * kLog2e;                       // G_L / 2 in log2 units
                                far = far || (-h0 > kRefLimit) || (-h1 > kRefLimit) || (-h2 > kRefLimit) || (-h3 > kRefLimit);
                                st_shared_f4(smem_u32(&M.vec[slot][32u * hf + 4u * m]), h0, h1, h2, h3);
                            }
                        }
                        const bool wide = __any_sync(0xffffffffu, far);
                        if (l == 0) M.wide[slot] = wide ? 1u : 0u;
                    }
                    uint32_t qo[16], ko[16];
#pragma unroll
                    for (uint32_t m = 0; m < 4; ++m) {
                        const uint4 qr = ld_shared_v4(sw_unit(tq, rho, 4u * hf + m)), kr = ld_shared_v4(sw_unit(tk, rho, 4u * hf + m));
                        const uint32_t qu[4] = {qr.x, qr.y, qr.z, qr.w}, ku[4] = {kr.x, kr.y, kr.z, kr.w};
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const float a0 = x[8 * m + 2 * e], a1 = x[8 * m + 2 * e + 1];
                            qo[4 * m + e] = hmul2_u32(qu[e], pack_half2(ex2(fmaf(a0, kLog2e, hq)), ex2(fmaf(a1, kLog2e, hq))));
                            ko[4 * m + e] = hmul2_u32(ku[e], pack_half2(ex2(fmaf(a0, -kLog2e, hk)), ex2(fmaf(a1, -kLog2e, hk))));
                        }
                    }
                    named_bar_sync(bar_id, kTeamThreads);             // the exact-path flag is known to the whole team
                    const bool wide = M.wide[slot] != 0u;
                    if (wide) {
                        gate_wide_chunk(rev, P.q_exp, P.q_mul, stage, tmT, tw, l, bar_id);
                    } else {
#pragma unroll
                        for (uint32_t m = 0; m < 4; ++m) {
                            st_shared_v4(sw_unit(tq, rho, 4u * hf + m), qo[4 * m], qo[4 * m + 1], qo[4 * m + 2], qo[4 * m + 3]);
                            st_shared_v4(sw_unit(tk, rho, 4u * hf + m), ko[4 * m], ko[4 * m + 1], ko[4 * m + 2], ko[4 * m + 3]);
                        }
                    }
                    fence_proxy_async_smem();
                    tc_fence_before();
                    named_bar_sync(bar_id, kTeamThreads);             // qt, kt are in place (and the outputs of the team's last chunk read)
                    GLA_EV(41);
                    if (issuer) {
                        tc_fence_after();
                        if (elect_one()) {
                            if (!wide) {
                                const uint64_t dQ = umma_desc_sw128(tq), dK = umma_desc_sw128(tk);
#pragma unroll
                                for (uint32_t ks = 0; ks < 4; ++ks) umma_f16(tmT, dQ + ks * 2u, dK + ks * 2u, idA, ks);
                            }
                            umma_commit(smem_u32(&M.a_done[team]));      // exact path: the team wrote the accumulator itself
                        }
                        __syncwarp();
                        if (ctr >= 2u) mbar_wait(ctx, &M.inc_free[(ctr - 2u) & 3u], ((ctr - 2u) >> 2) & 1u);        // state group has read this buffer's previous use
                        tc_fence_after();
                        if (elect_one()) {
                            const uint64_t dk = umma_desc_sw128(tk, 8192), dv = umma_desc_sw128(stage + 3 * kTileBytes, 8192);
                            const uint32_t tmI = tmem + kTmInc + 64u * p;
#pragma unroll
                            for (uint32_t ks = 0; ks < 4; ++ks) umma_f16(tmI, dk + ks * 128u, dv + ks * 128u, idS, ks);
                            umma_commit(smem_u32(&M.inc_done[p]));
                            mbar_arrive(smem_u32(&M.ops_ready[s]));
                        }
                        __syncwarp();
                    }
                    // ---- scores: TMEM -> causal mask -> fp16 tile over the gate tile
                    // fused epilogue: this thread's half row of the chunk's output gate is asked for now, into L2
                    const uint4* gp = nullptr;
                    if (kGated) {
                        const int p0 = (it.first_chunk + i) * kChunk;
                        const int u = (rev ? (P.T - p0 - kChunk) : p0) + static_cast<int>(rho);   // position along the scan
                        if (u >= 0 && u < P.T) {
                            // the token read at this row of the chunk follows the same mapping as the TMA boxes
                            long long tok = u;
                            if (P.Wc > 1) {
                                const int cc = u / P.Hc, rr = u - cc * P.Hc;
                                tok = static_cast<long long>(rr) * P.Wc + cc;
                            }
                            gp = reinterpret_cast<const uint4*>(P.gate + it.b * P.gate_sb + tok * P.gate_st + it.h * P.gate_sh + j0);
                            prefetch_l2(gp);
                        }
                    }
                    group_wait(ctx, &M.a_done[team], oturn & 1u, tw, bar_id, kTeamThreads);
                    GLA_EV(10);
                    tc_fence_after();
                    tmem_half_row(tmem, tw, kTmT + 64u * team, x);
                    mask_and_store_scores(rev, tg, rho, j0, x);
                    fence_proxy_async_smem();
                    tc_fence_before();
                    if (storer && elect_one()) tma_store_wait_read();   // the team's output tile: its last store has read it
                    named_bar_sync(bar_id, kTeamThreads);
                    GLA_EV(11);
                    if (issuer) {
                        tc_fence_after();
                        const uint32_t j = k2 & 1u;
                        if (elect_one()) {
                            const uint64_t da16 = umma_desc_sw128(tg), dv = umma_desc_sw128(stage + 3 * kTileBytes, 8192);
#pragma unroll
                            for (uint32_t ks = 0; ks < 4; ++ks) umma_f16(tmT, da16 + ks * 2u, dv + ks * 128u, idO, ks);
                        }
                        __syncwarp();
                        mbar_wait(ctx, &M.s16_ready[k2 & 3u], (k2 >> 2) & 1u);
                        tc_fence_after();
                        if (elect_one()) {
                            const uint64_t dq = umma_desc_sw128(tq), dS16 = umma_desc_sw128(base + kOffS16 + j * kTileBytes, 8192);
#pragma unroll
                            for (uint32_t ks = 0; ks < 4; ++ks) umma_f16(tmT, dq + ks * 2u, dS16 + ks * 128u, idO, 1);
                            umma_commit(smem_u32(&M.o_done[team]));
                            umma_commit(smem_u32(&M.s16_free[j]));
                            umma_commit(smem_u32(&M.empty[s]));
                        }
                        __syncwarp();
                    }
                    // ---- outputs: TMEM -> epilogue -> fp16 output tile -> TMA store
                    group_wait(ctx, &M.o_done[team], oturn & 1u, tw, bar_id, kTeamThreads);
                    GLA_EV(16);
                    tc_fence_after();
                    tmem_half_row(tmem, tw, kTmT + 64u * team, x);
                    tc_fence_before();
                    if (!kGated) {
                        if (P.o_mul != 1.f) {         // scale not folded into q and k (zero, negative or not finite)
#pragma unroll
                            for (int e = 0; e < 32; ++e) x[e] *= P.o_mul;
                        }
                    } else {
                        // y = o * rsqrt(mean(o^2) + eps) * w * silu(gate): the two lanes of a row share its sum of squares
                        float s4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                        for (int e = 0; e < 32; ++e) s4[e & 3] = fmaf(x[e], x[e], s4[e & 3]);
                        float ss = (s4[0] + s4[1]) + (s4[2] + s4[3]);
                        ss += __shfl_xor_sync(0xffffffffu, ss, 16);
                        const float rinv = P.o_mul * rsqrtf(ss * (P.o_mul * P.o_mul) * (1.f / kD) + P.rms_eps);
                        if (gp != nullptr) {       // rows past the end of the sequence are never sent out
                            const uint4* wp = reinterpret_cast<const uint4*>(P.rms_w + j0);
#pragma unroll
                            for (uint32_t m = 0; m < 4; ++m) {
                                const uint4 g4 = __ldg(gp + m), w4 = __ldg(wp + m);
                                const uint32_t gu[4] = {g4.x, g4.y, g4.z, g4.w}, wu[4] = {w4.x, w4.y, w4.z, w4.w};
#pragma unroll
                                for (int q2 = 0; q2 < 4; ++q2) {
                                    const float2 gf = unpack_half2(gu[q2]), wf = unpack_half2(wu[q2]);
                                    x[8 * m + 2 * q2] *= rinv * wf.x * silu_f(gf.x);
                                    x[8 * m + 2 * q2 + 1] *= rinv * wf.y * silu_f(gf.y);
                                }
                            }
                        }
                    }
                    store_row_f16<4>(out_tile, rho, j0 >> 3, x);
                    fence_proxy_async_smem();
                    named_bar_sync(bar_id, kTeamThreads);
                    GLA_EV(17);
                    if (storer && elect_one()) {
                        const BoxWalker bw(P, (it.first_chunk + i) * kChunk);
                        bw.for_each(P, [&](int id, int r, int c, int row) {
                            if (kL2Hints)
                                tma_store_5d_hint(&maps.m[TO][id], out_tile + static_cast<uint32_t>(row) * 128u, 0, it.h, r, c, it.b,
                                                  pol_stream);
                            else
                                tma_store_5d(&maps.m[TO][id], out_tile + static_cast<uint32_t>(row) * 128u, 0, it.h, r, c, it.b);
                        });
                        tma_store_commit();
                    }
                    __syncwarp();
                    ++oturn;
                    GLA_EV(13);
                }
            }
            __syncthreads();
        }
        if (storer && elect_one()) tma_store_wait_all();
    } else {
        // ==================================================================== service warps
        // These warps run their loops with all 32 lanes, in warp-uniform control flow, and only the issue of an
        // asynchronous instruction (TMA, tcgen05.mma, commit) is left to one elected lane.
        reg_budget<kRegsService>();
        while (true) {
            const int item = next_item();
            if (item >= P.num_items) break;
            const ItemInfo it = decode_item(P, item);
            const int npass = it.state_pass ? 2 : 1;
            if (w == kWarpProducer) {
                // ------------------------------------------------------------ TMA producer
                const uint64_t pol_keep = l2_policy_keep(), pol_stream = l2_policy_stream();
                for (int pass = 0; pass < npass; ++pass) {
                    const bool state_only = it.state_pass && pass == 0;
                    const bool back = state_only && kBackwardPrePass;
                    BoxWalker bw(P, (it.first_chunk + (back ? it.nchunks - 1 : 0)) * kChunk);
                    // tiles of a pre-pass are read again by the output pass; everything else is read once
                    const uint64_t pol = state_only ? pol_keep : pol_stream;
                    auto load = [&](uint32_t dst, int tensor, int id, uint32_t bar, int r, int c) {
                        if (kL2Hints) tma_load_5d_hint(dst, &maps.m[tensor][id], bar, 0, it.h, r, c, it.b, pol);
                        else tma_load_5d(dst, &maps.m[tensor][id], bar, 0, it.h, r, c, it.b);
                    };
                    for (int i = 0; i < it.nchunks; ++i, ++ctr) {
                        const uint32_t s = ctr % kNumStages, n = ctr / kNumStages;
                        mbar_wait(ctx, &M.empty[s], (n & 1u) ^ 1u);
                        GLA_EV(30);
                        if (elect_one()) {
                            const int ntens = state_only ? 3 : 4;
                            const uint32_t bar = smem_u32(&M.full[s]);
                            mbar_arrive_expect_tx(bar, static_cast<uint32_t>(kChunk * 128 * ntens));
                            const uint32_t stage = base + kOffStage + s * kStageBytes;
                            bw.for_each(P, [&](int id, int r, int c, int row) {
                                const uint32_t off = static_cast<uint32_t>(row) * 128u;
                                load(stage + 2 * kTileBytes + off, TG, id, bar, r, c);
                                load(stage + 1 * kTileBytes + off, TK, id, bar, r, c);
                                if (!state_only) load(stage + 0 * kTileBytes + off, TQ, id, bar, r, c);
                                load(stage + 3 * kTileBytes + off, TV, id, bar, r, c);
                            });
                            // rows the sequence does not have: boxes whose row coordinate lies past the column's end
                            // read nothing and fill their part of the tile with zeros
                            bw.for_each_missing(P, [&](int id, int row) {
                                const uint32_t off = static_cast<uint32_t>(row) * 128u;
                                tma_load_5d(stage + 2 * kTileBytes + off, &maps.m[TG][id], bar, 0, it.h, P.Hc, 0, it.b);
                                tma_load_5d(stage + 1 * kTileBytes + off, &maps.m[TK][id], bar, 0, it.h, P.Hc, 0, it.b);
                                if (!state_only)
                                    tma_load_5d(stage + 0 * kTileBytes + off, &maps.m[TQ][id], bar, 0, it.h, P.Hc, 0, it.b);
                                tma_load_5d(stage + 3 * kTileBytes + off, &maps.m[TV][id], bar, 0, it.h, P.Hc, 0, it.b);
                            });
                        }
                        __syncwarp();
                        if (back) bw.retreat(P);
                        else bw.advance(P);
                    }
                }
            } else if (w == kWarpX) {
                // ------------------------------------------------------------ gate-sum MMAs
                constexpr uint32_t idX = umma_idesc(FMT_F16, 0, 1, 64, 64);     // L (K-major) x g (rows = source rows)
                for (int pass = 0; pass < npass; ++pass) {
                    const bool state_only = it.state_pass && pass == 0;
                    const uint64_t dL = umma_desc_sw128(base + kOffLmat + (state_only ? kTileBytes : 0));
                    for (int i = 0; i < it.nchunks; ++i, ++ctr) {
                        const uint32_t s = ctr % kNumStages, team = ctr % kTeams, turn = ctr / kTeams;
                        if (logits) mbar_wait(ctx, &M.g_ready[s], (ctr / kNumStages) & 1u);
                        else mbar_wait(ctx, &M.full[s], (ctr / kNumStages) & 1u);
                        mbar_wait(ctx, &M.x_free[team], (turn & 1u) ^ 1u);          // the team has read its previous gate sums
                        tc_fence_after();
                        if (elect_one()) {
                            const uint64_t dg = umma_desc_sw128(base + kOffStage + s * kStageBytes + 2 * kTileBytes, 8192);
                            const uint32_t tmX = tmem + kTmX + 64u * team;
#pragma unroll
                            for (uint32_t ks = 0; ks < 4; ++ks) umma_f16(tmX, dL + ks * 2u, dg + ks * 128u, idX, ks);
                            umma_commit(smem_u32(&M.x_done[team]));
                        }
                        __syncwarp();
                        GLA_EV(20);
                    }
                }
            }
            __syncthreads();
        }
    }

    GLA_EV(4);
    tc_fence_before();
    __syncthreads();
    GLA_EV(7);
    GLA_EVV(8, globaltimer_ns());
    if (w == kWarpProducer) tmem_dealloc(tmem, kTmemCols);
}

}  // namespace gla
