// Gradient of the gated-linear-attention operator, token by token with the state in registers.
//
//   forward    S_t = exp(g_t) S_{t-1} + k_t v_t^T ,  o_t = scale q_t^T S_t
//   gradient   dS_t = exp(g_{t+1}) dS_{t+1} + scale q_t do_t^T
//              dq_t = scale S_t do_t     dk_t = dS_t v_t     dv_t = dS_t^T k_t
//              dg_t = sum_{s >= t} (q_s dq_s - k_s dk_s)   (+ the final state's term at the last token)
//
// The reference trains through the third-party FLA operator (engine/gtr/backbone/vit_adapter.py:441,560-568); its
// own CUDA extension has no gradient.  Three independent sweeps run as three kinds of CTA per (batch, head):
//   kind 0  walks forward with S and emits dq;
//   kind 1  walks backward with dS and emits dk (and d initial_state);
//   kind 2  walks backward with a second copy of dS, blocked the other way round, and emits dv.
// A thread owns a small block of the state, so a token costs it 6 or 7 shared-memory reads of 16 bytes, and every
// per-token reduction is inside the thread plus a 3-step butterfly over 8 lanes.  Tokens are staged 32 at a time:
// the next chunk's fp16 rows are fetched into registers while the current chunk is worked from fp32 tiles in
// shared memory.  A last kernel turns the per-token products q dq - k dk into dg by a reverse running sum.
// All arithmetic is fp32 on CUDA cores, two lanes per instruction (fma.rn.f32x2): 1.5 instructions per state element and
// token, so the sweeps are bound by instruction issue, not by memory.
#pragma once
#include <cuda_fp16.h>
#include <cstdint>

namespace gla {

constexpr int kBwdThreads = 128;
constexpr int kBwdChunk = 32;

struct BwdParams {
    const __half *q, *k, *v, *g, *d_o;
    __half *dq, *dk, *dv;
    float* dg;
    const float* h0;      // [B,H,K,64] or null
    const float* dht;     // [B,H,K,64] or null
    float* dh0;           // [B,H,K,64] or null
    float *qdq, *kdk;     // scratch [B,T,H,K]
    float* g_last;        // scratch [B,H,K]: sum_v dht * final_state
    float* seg_state;     // scratch [2][B*H][nseg][K,64]: a segment's own contribution (forward S, backward dS)
    float* seg_start;     // scratch, same shape: the state a segment starts from
    float* seg_decay;     // scratch [2][B*H][nseg][K]: product of the gates over a segment
    int B, T, H;
    int nseg, seg_len;    // a sequence is cut into nseg pieces of seg_len tokens (a multiple of 32), each its own CTA
    float scale;
};

// Two fp32 lanes per instruction (the packed FMA pipe of sm_100): the sweeps are bound by instruction issue.
__device__ __forceinline__ float2 bwd_fma2(float2 a, float2 b, float2 c) {
    unsigned long long d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d)
        : "l"(reinterpret_cast<const unsigned long long&>(a)), "l"(reinterpret_cast<const unsigned long long&>(b)),
          "l"(reinterpret_cast<const unsigned long long&>(c)));
    return reinterpret_cast<const float2&>(d);
}
__device__ __forceinline__ float2 bwd_mul2(float2 a, float2 b) {
    unsigned long long d;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d)
        : "l"(reinterpret_cast<const unsigned long long&>(a)), "l"(reinterpret_cast<const unsigned long long&>(b)));
    return reinterpret_cast<const float2&>(d);
}

// 32 tokens x W halves of one head, 16 bytes per thread and step; rows past the sequence read as zero, which makes
// a padded token the identity (gate 1, no update).
template <int W>
__device__ __forceinline__ void bwd_fetch(uint4 (&r)[W / 32], const __half* base, int64_t tok_stride, int t0, int T, int tid) {
#pragma unroll
    for (int i = 0; i < W / 32; ++i) {
        const int idx = tid + kBwdThreads * i, row = idx / (W / 8), c8 = idx % (W / 8), t = t0 + row;
        r[i] = t < T ? __ldg(reinterpret_cast<const uint4*>(base + t * tok_stride + c8 * 8)) : make_uint4(0u, 0u, 0u, 0u);
    }
}

template <int W, bool kExp>
__device__ __forceinline__ void bwd_spread(float* tile, const uint4 (&r)[W / 32], float mul, int tid) {
#pragma unroll
    for (int i = 0; i < W / 32; ++i) {
        const int idx = tid + kBwdThreads * i, row = idx / (W / 8), c8 = idx % (W / 8);
        const __half2* h = reinterpret_cast<const __half2*>(&r[i]);
        float f[8];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float2 x = __half22float2(h[e]);
            f[2 * e] = kExp ? __expf(x.x) : x.x * mul;
            f[2 * e + 1] = kExp ? __expf(x.y) : x.y * mul;
        }
        float4* dst = reinterpret_cast<float4*>(tile + row * W + c8 * 8);
        dst[0] = make_float4(f[0], f[1], f[2], f[3]);
        dst[1] = make_float4(f[4], f[5], f[6], f[7]);
    }
}

template <int W>
__device__ __forceinline__ void bwd_keep(__half* tile, const uint4 (&r)[W / 32], int tid) {
#pragma unroll
    for (int i = 0; i < W / 32; ++i) {
        const int idx = tid + kBwdThreads * i;
        reinterpret_cast<uint4*>(tile)[idx] = r[i];
    }
}

struct BwdSmem {
    float tile[4][kBwdChunk * 64];
    float out[kBwdChunk * 64];
    __half raw[kBwdChunk * 64];
};

// Sum over the 8 lanes of a group (lane bits 0..2) of R values each lane holds, by a butterfly that halves the values
// kept at every exchange: 4 shuffles for R = 4, 3 for R = 2.  Every lane ends with the complete sum of value `which`.
template <int R>
__device__ __forceinline__ float bwd_reduce8(const float (&v)[R], int lane, int& which) {
    constexpr unsigned kAll = 0xffffffffu;
    const bool b2 = (lane & 4) != 0, b1 = (lane & 2) != 0;
    float k;
    if (R == 4) {
        float k0 = b2 ? v[R - 2] : v[0], k1 = b2 ? v[R - 1] : v[1];
        const float s0 = b2 ? v[0] : v[R - 2], s1 = b2 ? v[1] : v[R - 1];
        k0 += __shfl_xor_sync(kAll, s0, 4);
        k1 += __shfl_xor_sync(kAll, s1, 4);
        k = b1 ? k1 : k0;
        k += __shfl_xor_sync(kAll, b1 ? k0 : k1, 2);
        which = (b2 ? 2 : 0) + (b1 ? 1 : 0);
    } else {
        k = b2 ? v[R - 1] : v[0];
        k += __shfl_xor_sync(kAll, b2 ? v[0] : v[R - 1], 4);
        k += __shfl_xor_sync(kAll, k, 2);
        which = b2 ? 1 : 0;
    }
    k += __shfl_xor_sync(kAll, k, 1);
    return k;
}

template <int N>
__device__ __forceinline__ void bwd_lds(float (&d)[N], const float* src) {
    if (N == 2) {
        const float2 u = *reinterpret_cast<const float2*>(src);
        d[0] = u.x; d[1] = u.y;
    } else {
#pragma unroll
        for (int i = 0; i < N / 4; ++i) {
            const float4 u = reinterpret_cast<const float4*>(src)[i];
            d[4 * i] = u.x; d[4 * i + 1] = u.y; d[4 * i + 2] = u.z; d[4 * i + 3] = u.w;
        }
    }
}

// Kinds 0 and 1.  A thread owns an R x 8 block of the K x 64 state (R = K / 16): 16 row groups x 8 column groups, the 8
// column groups of a row group in neighbouring lanes.  Per token it reads its R gates and key-side factors and its 8 + 8
// value-side entries (6 shared-memory reads of 16 bytes), and the R row sums are completed across the 8 lanes.
//   kind 0 (forward in t):   S = a S + b x ,  acc = S . y     a = exp(g_t), b = k_t,        x = v_t,  y = do_t
//   kind 1 (backward in t):  S = S + b x ,    acc = S . y ,  S = a S     a = exp(g_t), b = scale q_t, x = do_t, y = v_t
// With kStateOnly the sweep starts from zero, emits nothing per token and leaves the segment's own contribution to the
// state, and the product of its gates, for gla_bwd_combine_kernel.
template <int K, int kKind, bool kStateOnly>
__device__ void bwd_row_sweep(const BwdParams& P, BwdSmem& sm, int bh, int seg) {
    constexpr int R = K / 16;
    constexpr bool kFwd = kKind == 0;
    const int tid = threadIdx.x, lane = tid & 31, cg = tid & 7, rg = tid >> 3;
    const int b = bh / P.H, h = bh % P.H;
    const int t_begin = seg * P.seg_len, T = min(P.T, t_begin + P.seg_len);        // this CTA's tokens: [t_begin, T)
    const int64_t strideK = static_cast<int64_t>(P.H) * K, strideV = static_cast<int64_t>(P.H) * 64;
    const int64_t offK = (static_cast<int64_t>(b) * P.T * P.H + h) * K, offV = (static_cast<int64_t>(b) * P.T * P.H + h) * 64;
    const __half* pa = P.g + offK;                                  // gate
    const __half* pb = (kFwd ? P.k : P.q) + offK;                   // the rank-one update's key-side factor
    const __half* px = (kFwd ? P.v : P.d_o) + offV;                 // its value-side factor
    const __half* py = (kFwd ? P.d_o : P.v) + offV;                 // what the state is contracted with
    const __half* pr = (kFwd ? P.q : P.k) + offK;                   // the factor of the gate-gradient product
    __half* pout = (kFwd ? P.dq : P.dk) + offK;
    float* pprod = (kFwd ? P.qdq : P.kdk) + offK;
    const int block_off = R * rg * 64 + 8 * cg;                     // this thread's block inside a [K,64] state
    const int64_t state_off = static_cast<int64_t>(bh) * K * 64 + block_off;
    const int64_t seg_slot = (static_cast<int64_t>(kFwd ? 0 : P.B * P.H) + bh) * P.nseg + seg;

    float2 S[R][4];
    float decay[R];
    const float* init = kStateOnly ? nullptr
                        : P.nseg > 1 ? P.seg_start + seg_slot * K * 64 + block_off
                        : (kFwd ? P.h0 : P.dht) ? (kFwd ? P.h0 : P.dht) + state_off : nullptr;
#pragma unroll
    for (int r = 0; r < R; ++r) {
        decay[r] = 1.f;
#pragma unroll
        for (int c = 0; c < 4; ++c)
            S[r][c] = init ? *reinterpret_cast<const float2*>(init + r * 64 + 2 * c) : make_float2(0.f, 0.f);
    }

    const int nchunks = (T - t_begin + kBwdChunk - 1) / kBwdChunk;
    uint4 ra[K / 32], rb[K / 32], rr[K / 32], rx[2], ry[2];
    auto fetch = [&](int ci) {
        const int t0 = t_begin + (kFwd ? ci : nchunks - 1 - ci) * kBwdChunk;
        bwd_fetch<K>(ra, pa, strideK, t0, T, tid);
        bwd_fetch<K>(rb, pb, strideK, t0, T, tid);
        bwd_fetch<64>(rx, px, strideV, t0, T, tid);
        if (!kStateOnly) {
            bwd_fetch<K>(rr, pr, strideK, t0, T, tid);
            bwd_fetch<64>(ry, py, strideV, t0, T, tid);
        }
    };
    if (nchunks > 0) fetch(0);
    for (int ci = 0; ci < nchunks; ++ci) {
        const int t0 = t_begin + (kFwd ? ci : nchunks - 1 - ci) * kBwdChunk;
        bwd_spread<K, true>(sm.tile[0], ra, 1.f, tid);
        bwd_spread<K, false>(sm.tile[1], rb, kFwd ? 1.f : P.scale, tid);
        bwd_spread<64, false>(sm.tile[2], rx, 1.f, tid);
        if (!kStateOnly) {
            bwd_spread<64, false>(sm.tile[3], ry, 1.f, tid);
            bwd_keep<K>(sm.raw, rr, tid);
        }
        __syncthreads();
        if (ci + 1 < nchunks) fetch(ci + 1);
#pragma unroll 4
        for (int tt = 0; tt < kBwdChunk; ++tt) {
            const int t = kFwd ? tt : kBwdChunk - 1 - tt;
            float a[R], bq[R], x[8], y[8], v[R];
            bwd_lds<R>(a, &sm.tile[0][t * K + R * rg]);
            bwd_lds<R>(bq, &sm.tile[1][t * K + R * rg]);
            bwd_lds<8>(x, &sm.tile[2][t * 64 + 8 * cg]);
            if (kStateOnly) {
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    const float2 aa = make_float2(a[r], a[r]), bb = make_float2(bq[r], bq[r]);
                    decay[r] *= a[r];
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        const float2 x2 = make_float2(x[2 * c], x[2 * c + 1]);
                        if (kFwd) S[r][c] = bwd_fma2(S[r][c], aa, bwd_mul2(bb, x2));
                        else S[r][c] = bwd_mul2(bwd_fma2(bb, x2, S[r][c]), aa);
                    }
                }
                continue;
            }
            bwd_lds<8>(y, &sm.tile[3][t * 64 + 8 * cg]);
#pragma unroll
            for (int r = 0; r < R; ++r) {
                const float2 aa = make_float2(a[r], a[r]), bb = make_float2(bq[r], bq[r]);
                float2 acc = make_float2(0.f, 0.f);
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const float2 x2 = make_float2(x[2 * c], x[2 * c + 1]), y2 = make_float2(y[2 * c], y[2 * c + 1]);
                    if (kFwd) S[r][c] = bwd_fma2(S[r][c], aa, bwd_mul2(bb, x2));
                    else S[r][c] = bwd_fma2(bb, x2, S[r][c]);
                    acc = bwd_fma2(S[r][c], y2, acc);
                    if (!kFwd) S[r][c] = bwd_mul2(S[r][c], aa);
                }
                v[r] = acc.x + acc.y;
            }
            int which;
            const float sum = bwd_reduce8<R>(v, lane, which);
            if (!(lane & 1)) sm.out[t * K + R * rg + which] = sum;
        }
        if (kStateOnly) {
            __syncthreads();
            continue;
        }
        __syncthreads();
        // the chunk's gradient rows, and their products with q (k) for the gate gradient
#pragma unroll
        for (int i = 0; i < K / 32; ++i) {
            const int idx = tid + kBwdThreads * i, r = idx / (K / 8), c8 = idx % (K / 8), t = t0 + r;
            if (t < T) {
                const float4 u0 = *reinterpret_cast<const float4*>(&sm.out[r * K + c8 * 8]);
                const float4 u1 = *reinterpret_cast<const float4*>(&sm.out[r * K + c8 * 8 + 4]);
                const float mul = kFwd ? P.scale : 1.f;
                const float d[8] = {u0.x * mul, u0.y * mul, u0.z * mul, u0.w * mul, u1.x * mul, u1.y * mul, u1.z * mul, u1.w * mul};
                const uint4 rw = reinterpret_cast<const uint4*>(sm.raw)[idx];
                const __half2* hr = reinterpret_cast<const __half2*>(&rw);
                uint4 packed;
                __half2* hp = reinterpret_cast<__half2*>(&packed);
                float pr8[8];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float2 f = __half22float2(hr[e]);
                    hp[e] = __floats2half2_rn(d[2 * e], d[2 * e + 1]);
                    pr8[2 * e] = f.x * d[2 * e];
                    pr8[2 * e + 1] = f.y * d[2 * e + 1];
                }
                *reinterpret_cast<uint4*>(pout + t * strideK + c8 * 8) = packed;
                float4* pp = reinterpret_cast<float4*>(pprod + t * strideK + c8 * 8);
                pp[0] = make_float4(pr8[0], pr8[1], pr8[2], pr8[3]);
                pp[1] = make_float4(pr8[4], pr8[5], pr8[6], pr8[7]);
            }
        }
        __syncthreads();
    }
    if (kStateOnly) {
#pragma unroll
        for (int r = 0; r < R; ++r) {
#pragma unroll
            for (int c = 0; c < 4; ++c)
                *reinterpret_cast<float2*>(P.seg_state + seg_slot * K * 64 + block_off + r * 64 + 2 * c) = S[r][c];
            if (cg == 0) P.seg_decay[seg_slot * K + R * rg + r] = decay[r];
        }
    } else if (kFwd) {
        if (P.g_last && seg == P.nseg - 1) {                      // S is the final state here
            float v[R];
#pragma unroll
            for (int r = 0; r < R; ++r) {
                float acc = 0.f;
                if (P.dht) {
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        const float2 d = *reinterpret_cast<const float2*>(P.dht + state_off + r * 64 + 2 * c);
                        acc = fmaf(d.x, S[r][c].x, fmaf(d.y, S[r][c].y, acc));
                    }
                }
                v[r] = acc;
            }
            int which;
            const float sum = bwd_reduce8<R>(v, lane, which);
            if (!(lane & 1)) P.g_last[static_cast<int64_t>(bh) * K + R * rg + which] = sum;
        }
    } else if (P.dh0 && seg == 0) {
#pragma unroll
        for (int r = 0; r < R; ++r)
#pragma unroll
            for (int c = 0; c < 4; ++c) *reinterpret_cast<float2*>(P.dh0 + state_off + r * 64 + 2 * c) = S[r][c];
    }
}

// Kind 2.  A thread owns a (K / 8) x 4 block of dS: 8 row groups in neighbouring lanes x 16 column groups.  Its rows are
// 4 rg .. 4 rg + 3 (and 32 + the same for K = 64), so that the 8 lanes' 16-byte reads of the key-side tiles fall on distinct
// banks.  The 4 column sums are completed across the 8 lanes.
//   S = S + bq x ,  acc = S^T kk ,  S = a S      a = exp(g_t), bq = scale q_t, kk = k_t (over the rows),  x = do_t (over the columns)
template <int K>
__device__ void bwd_col_sweep(const BwdParams& P, BwdSmem& sm, int bh, int seg) {
    constexpr int RC = K / 8;
    const int tid = threadIdx.x, lane = tid & 31, rg = tid & 7, cg = tid >> 3;
    const int b = bh / P.H, h = bh % P.H;
    const int t_begin = seg * P.seg_len, T = min(P.T, t_begin + P.seg_len);
    const int64_t strideK = static_cast<int64_t>(P.H) * K, strideV = static_cast<int64_t>(P.H) * 64;
    const int64_t offK = (static_cast<int64_t>(b) * P.T * P.H + h) * K, offV = (static_cast<int64_t>(b) * P.T * P.H + h) * 64;
    const __half *pa = P.g + offK, *pq = P.q + offK, *pk = P.k + offK, *px = P.d_o + offV;
    __half* pout = P.dv + offV;

    float2 S[RC][2];
    const float* init = P.nseg > 1 ? P.seg_start + ((static_cast<int64_t>(P.B) * P.H + bh) * P.nseg + seg) * K * 64
                        : P.dht ? P.dht + static_cast<int64_t>(bh) * K * 64 : nullptr;
#pragma unroll
    for (int r = 0; r < RC; ++r) {
        const int row = (r / 4) * 32 + 4 * rg + (r % 4);
#pragma unroll
        for (int c = 0; c < 2; ++c)
            S[r][c] = init ? *reinterpret_cast<const float2*>(init + row * 64 + 4 * cg + 2 * c) : make_float2(0.f, 0.f);
    }

    const int nchunks = (T - t_begin + kBwdChunk - 1) / kBwdChunk;
    uint4 ra[K / 32], rq[K / 32], rk[K / 32], rx[2];
    auto fetch = [&](int ci) {
        const int t0 = t_begin + (nchunks - 1 - ci) * kBwdChunk;
        bwd_fetch<K>(ra, pa, strideK, t0, T, tid);
        bwd_fetch<K>(rq, pq, strideK, t0, T, tid);
        bwd_fetch<K>(rk, pk, strideK, t0, T, tid);
        bwd_fetch<64>(rx, px, strideV, t0, T, tid);
    };
    if (nchunks > 0) fetch(0);
    for (int ci = 0; ci < nchunks; ++ci) {
        const int t0 = t_begin + (nchunks - 1 - ci) * kBwdChunk;
        bwd_spread<K, true>(sm.tile[0], ra, 1.f, tid);
        bwd_spread<K, false>(sm.tile[1], rq, P.scale, tid);
        bwd_spread<K, false>(sm.tile[2], rk, 1.f, tid);
        bwd_spread<64, false>(sm.tile[3], rx, 1.f, tid);
        __syncthreads();
        if (ci + 1 < nchunks) fetch(ci + 1);
#pragma unroll 4
        for (int tt = 0; tt < kBwdChunk; ++tt) {
            const int t = kBwdChunk - 1 - tt;
            float a[RC], qq[RC], kk[RC], x[4];
#pragma unroll
            for (int i = 0; i < RC / 4; ++i) {
                bwd_lds<4>(reinterpret_cast<float(&)[4]>(a[4 * i]), &sm.tile[0][t * K + 32 * i + 4 * rg]);
                bwd_lds<4>(reinterpret_cast<float(&)[4]>(qq[4 * i]), &sm.tile[1][t * K + 32 * i + 4 * rg]);
                bwd_lds<4>(reinterpret_cast<float(&)[4]>(kk[4 * i]), &sm.tile[2][t * K + 32 * i + 4 * rg]);
            }
            bwd_lds<4>(x, &sm.tile[3][t * 64 + 4 * cg]);
            const float2 x2[2] = {make_float2(x[0], x[1]), make_float2(x[2], x[3])};
            float2 acc[2] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
#pragma unroll
            for (int r = 0; r < RC; ++r) {
                const float2 q2 = make_float2(qq[r], qq[r]), k2 = make_float2(kk[r], kk[r]), a2 = make_float2(a[r], a[r]);
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    S[r][c] = bwd_fma2(q2, x2[c], S[r][c]);
                    acc[c] = bwd_fma2(S[r][c], k2, acc[c]);
                    S[r][c] = bwd_mul2(S[r][c], a2);
                }
            }
            const float v[4] = {acc[0].x, acc[0].y, acc[1].x, acc[1].y};
            int which;
            const float sum = bwd_reduce8<4>(v, lane, which);
            if (!(lane & 1)) sm.out[t * 64 + 4 * cg + which] = sum;
        }
        __syncthreads();
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int idx = tid + kBwdThreads * i, r = idx / 8, c8 = idx % 8, t = t0 + r;
            if (t < T) {
                const float4 u0 = *reinterpret_cast<const float4*>(&sm.out[r * 64 + c8 * 8]);
                const float4 u1 = *reinterpret_cast<const float4*>(&sm.out[r * 64 + c8 * 8 + 4]);
                uint4 packed;
                __half2* hp = reinterpret_cast<__half2*>(&packed);
                hp[0] = __floats2half2_rn(u0.x, u0.y); hp[1] = __floats2half2_rn(u0.z, u0.w);
                hp[2] = __floats2half2_rn(u1.x, u1.y); hp[3] = __floats2half2_rn(u1.z, u1.w);
                *reinterpret_cast<uint4*>(pout + t * strideV + c8 * 8) = packed;
            }
        }
        __syncthreads();
    }
}

template <int K>
__global__ void __launch_bounds__(kBwdThreads) gla_bwd_sweep_kernel(const BwdParams P) {
    __shared__ __align__(16) BwdSmem sm;
    const int bh = blockIdx.x / P.nseg, seg = blockIdx.x % P.nseg, kind = blockIdx.y;
    if (kind == 0) bwd_row_sweep<K, 0, false>(P, sm, bh, seg);
    else if (kind == 1) bwd_row_sweep<K, 1, false>(P, sm, bh, seg);
    else bwd_col_sweep<K>(P, sm, bh, seg);
}

// Sequences cut into segments (few sequences, many tokens): every segment but the last in sweep order first runs alone
// from a zero state (this kernel: S of segments 0 .. nseg-2 forward, dS of segments 1 .. nseg-1 backward) ...
template <int K>
__global__ void __launch_bounds__(kBwdThreads) gla_bwd_state_kernel(const BwdParams P) {
    __shared__ __align__(16) BwdSmem sm;
    const int bh = blockIdx.x / (P.nseg - 1), i = blockIdx.x % (P.nseg - 1);
    if (blockIdx.y == 0) bwd_row_sweep<K, 0, true>(P, sm, bh, i);
    else bwd_row_sweep<K, 1, true>(P, sm, bh, i + 1);
}

// ... then the segments' contributions are chained, S' = decay * S + own, into the state each segment starts from
// (seg_start, laid out like seg_state), which gla_bwd_sweep_kernel picks up.  blockIdx.y: 0 forward states, 1 backward;
// one state element per thread, so the loads of a thread do not depend on one another.
template <int K>
__global__ void __launch_bounds__(256) gla_bwd_combine_kernel(const BwdParams P) {
    const int bh = blockIdx.x, back = blockIdx.y, nseg = P.nseg;
    const int e = blockIdx.z * 256 + threadIdx.x, row = e / 64;
    const int64_t slot0 = (static_cast<int64_t>(back ? P.B * P.H : 0) + bh) * nseg;
    const float* __restrict__ own = P.seg_state + slot0 * K * 64 + e;
    float* __restrict__ start = P.seg_start + slot0 * K * 64 + e;
    const float* __restrict__ dec = P.seg_decay + slot0 * K + row;
    const float* init = back ? P.dht : P.h0;
    float S = init ? init[static_cast<int64_t>(bh) * K * 64 + e] : 0.f;
    if (!back) {
#pragma unroll 4
        for (int j = 0; j < nseg - 1; ++j) {
            start[static_cast<int64_t>(j) * K * 64] = S;
            S = fmaf(__ldg(dec + j * K), S, __ldg(own + static_cast<int64_t>(j) * K * 64));
        }
        start[static_cast<int64_t>(nseg - 1) * K * 64] = S;
    } else {
#pragma unroll 4
        for (int j = nseg - 1; j > 0; --j) {
            start[static_cast<int64_t>(j) * K * 64] = S;
            S = fmaf(__ldg(dec + j * K), S, __ldg(own + static_cast<int64_t>(j) * K * 64));
        }
        start[0] = S;
    }
}

// dg_t = sum_{s >= t} (q_s dq_s - k_s dk_s), per (batch, head, channel).  One CTA per (batch, head, kCh channels):
// 1024 / kCh slices of the sequence, each summed on its own first, then walked backwards from the total of the slices
// after it.  kCh = K reads whole rows (many sequences); kCh = 16 gives four times the CTAs (few, long sequences).
template <int K, int kCh>
__global__ void __launch_bounds__(1024) gla_bwd_dg_kernel(const BwdParams P) {
    constexpr int kSlices = 1024 / kCh;
    __shared__ float total[kSlices][kCh];
    const int bh = blockIdx.x, b = bh / P.H, h = bh % P.H, T = P.T;
    const int cl = threadIdx.x % kCh, c = blockIdx.y * kCh + cl, s = threadIdx.x / kCh;
    const int64_t stride = static_cast<int64_t>(P.H) * K, off = (static_cast<int64_t>(b) * T * P.H + h) * K + c;
    const float* __restrict__ pq = P.qdq + off;
    const float* __restrict__ pk = P.kdk + off;
    float* __restrict__ pg = P.dg + off;
    const int per = (T + kSlices - 1) / kSlices, lo = s * per, hi = min(T, lo + per);
    const float last = P.g_last ? P.g_last[static_cast<int64_t>(bh) * K + c] : 0.f;
    float sum = 0.f;
#pragma unroll 8
    for (int t = lo; t < hi; ++t) sum += __ldg(pq + t * stride) - __ldg(pk + t * stride);
    if (lo < T && hi == T) sum += last;
    total[s][cl] = sum;
    __syncthreads();
    float run = 0.f;
    for (int j = s + 1; j < kSlices; ++j) run += total[j][cl];
    if (lo < T && hi == T) run += last;
#pragma unroll 8
    for (int t = hi - 1; t >= lo; --t) {
        run += __ldg(pq + t * stride) - __ldg(pk + t * stride);
        pg[t * stride] = run;
    }
}

}  // namespace gla
