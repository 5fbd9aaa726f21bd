// Gradient of the gated-linear-attention operator, token by token with the state in registers.
//
//   forward    S_t = exp(g_t) S_{t-1} + k_t v_t^T ,  o_t = scale q_t^T S_t
//   gradient   dS_t = exp(g_{t+1}) dS_{t+1} + scale q_t do_t^T
//              dq_t = scale S_t do_t     dk_t = dS_t v_t     dv_t = dS_t^T k_t
//              dg_t = sum_{s >= t} (q_s dq_s - k_s dk_s)   (+ the final state's term at the last token)
//
// The reference trains through the third-party FLA operator (engine/gtr/backbone/vit_adapter.py:441,560-568); its
// own CUDA extension has no gradient.  Three independent sweeps run as three kinds of CTA per (batch, head):
//   kind 0  walks forward with S (a thread owns one key row and a slice of the value columns) and emits dq;
//   kind 1  walks backward with dS in the same ownership and emits dk (and d initial_state);
//   kind 2  walks backward with a second copy of dS owned by value column, and emits dv,
// so that every per-token reduction is inside a thread plus one or two shuffles.  Tokens are staged 32 at a time:
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
    int B, T, H;
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

// Kinds 0 and 1.  A thread owns row `row` of the K x 64 state and NV of its columns.
//   kind 0 (forward in t):   S = a S + b x ,  acc = S . y     a = exp(g_t), b = k_t,        x = v_t,  y = do_t
//   kind 1 (backward in t):  S = S + b x ,    acc = S . y ,  S = a S     a = exp(g_t), b = scale q_t, x = do_t, y = v_t
template <int K, int kKind>
__device__ void bwd_row_sweep(const BwdParams& P, BwdSmem& sm, int bh) {
    constexpr int kParts = kBwdThreads / K, NV = 64 / kParts;
    constexpr bool kFwd = kKind == 0;
    const int tid = threadIdx.x, row = tid / kParts, part = tid % kParts;
    const int b = bh / P.H, h = bh % P.H, T = P.T;
    const int64_t strideK = static_cast<int64_t>(P.H) * K, strideV = static_cast<int64_t>(P.H) * 64;
    const int64_t offK = (static_cast<int64_t>(b) * T * P.H + h) * K, offV = (static_cast<int64_t>(b) * T * P.H + h) * 64;
    const __half* pa = P.g + offK;                                  // gate
    const __half* pb = (kFwd ? P.k : P.q) + offK;                   // the rank-one update's key-side factor
    const __half* px = (kFwd ? P.v : P.d_o) + offV;                 // its value-side factor
    const __half* py = (kFwd ? P.d_o : P.v) + offV;                 // what the state is contracted with
    const __half* pr = (kFwd ? P.q : P.k) + offK;                   // the factor of the gate-gradient product
    __half* pout = (kFwd ? P.dq : P.dk) + offK;
    float* pprod = (kFwd ? P.qdq : P.kdk) + offK;

    float2 S[NV / 2];
    const float* init = kFwd ? P.h0 : P.dht;
#pragma unroll
    for (int j = 0; j < NV / 2; ++j) {
        const float* src = init + (static_cast<int64_t>(bh) * K + row) * 64 + part * NV + 2 * j;
        S[j] = init ? make_float2(src[0], src[1]) : make_float2(0.f, 0.f);
    }

    const int nchunks = (T + kBwdChunk - 1) / kBwdChunk;
    uint4 ra[K / 32], rb[K / 32], rr[K / 32], rx[2], ry[2];
    auto fetch = [&](int ci) {
        const int t0 = (kFwd ? ci : nchunks - 1 - ci) * kBwdChunk;
        bwd_fetch<K>(ra, pa, strideK, t0, T, tid);
        bwd_fetch<K>(rb, pb, strideK, t0, T, tid);
        bwd_fetch<K>(rr, pr, strideK, t0, T, tid);
        bwd_fetch<64>(rx, px, strideV, t0, T, tid);
        bwd_fetch<64>(ry, py, strideV, t0, T, tid);
    };
    if (nchunks > 0) fetch(0);
    for (int ci = 0; ci < nchunks; ++ci) {
        const int t0 = (kFwd ? ci : nchunks - 1 - ci) * kBwdChunk;
        bwd_spread<K, true>(sm.tile[0], ra, 1.f, tid);
        bwd_spread<K, false>(sm.tile[1], rb, kFwd ? 1.f : P.scale, tid);
        bwd_spread<64, false>(sm.tile[2], rx, 1.f, tid);
        bwd_spread<64, false>(sm.tile[3], ry, 1.f, tid);
        bwd_keep<K>(sm.raw, rr, tid);
        __syncthreads();
        if (ci + 1 < nchunks) fetch(ci + 1);
#pragma unroll 2
        for (int tt = 0; tt < kBwdChunk; ++tt) {
            const int t = kFwd ? tt : kBwdChunk - 1 - tt;
            const float a = sm.tile[0][t * K + row], bq = sm.tile[1][t * K + row];
            const float4* X = reinterpret_cast<const float4*>(&sm.tile[2][t * 64 + part * NV]);
            const float4* Y = reinterpret_cast<const float4*>(&sm.tile[3][t * 64 + part * NV]);
            const float2 aa = make_float2(a, a), bb = make_float2(bq, bq);
            float2 acc2 = make_float2(0.f, 0.f);
#pragma unroll
            for (int j = 0; j < NV / 4; ++j) {
                const float4 x = X[j], y = Y[j];
                const float2 x0 = make_float2(x.x, x.y), x1 = make_float2(x.z, x.w);
                const float2 y0 = make_float2(y.x, y.y), y1 = make_float2(y.z, y.w);
                if (kFwd) {
                    S[2 * j] = bwd_fma2(S[2 * j], aa, bwd_mul2(bb, x0));
                    S[2 * j + 1] = bwd_fma2(S[2 * j + 1], aa, bwd_mul2(bb, x1));
                } else {
                    S[2 * j] = bwd_fma2(bb, x0, S[2 * j]);
                    S[2 * j + 1] = bwd_fma2(bb, x1, S[2 * j + 1]);
                }
                acc2 = bwd_fma2(S[2 * j], y0, acc2);
                acc2 = bwd_fma2(S[2 * j + 1], y1, acc2);
                if (!kFwd) {
                    S[2 * j] = bwd_mul2(S[2 * j], aa);
                    S[2 * j + 1] = bwd_mul2(S[2 * j + 1], aa);
                }
            }
            float acc = acc2.x + acc2.y;
            acc += __shfl_xor_sync(0xffffffffu, acc, 1);
            if (kParts == 4) acc += __shfl_xor_sync(0xffffffffu, acc, 2);
            if (part == 0) sm.out[t * K + row] = acc;
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
    if (kFwd) {
        if (P.g_last) {                      // S is the final state here
            float acc = 0.f;
            if (P.dht) {
#pragma unroll
                for (int j = 0; j < NV / 2; ++j) {
                    const float* d = P.dht + (static_cast<int64_t>(bh) * K + row) * 64 + part * NV + 2 * j;
                    acc = fmaf(d[0], S[j].x, fmaf(d[1], S[j].y, acc));
                }
            }
            acc += __shfl_xor_sync(0xffffffffu, acc, 1);
            if (kParts == 4) acc += __shfl_xor_sync(0xffffffffu, acc, 2);
            if (part == 0) P.g_last[static_cast<int64_t>(bh) * K + row] = acc;
        }
    } else if (P.dh0) {
#pragma unroll
        for (int j = 0; j < NV / 2; ++j)
            *reinterpret_cast<float2*>(P.dh0 + (static_cast<int64_t>(bh) * K + row) * 64 + part * NV + 2 * j) = S[j];
    }
}

// Kind 2.  A thread owns value column `col` of dS and NC of its key rows:
//   S = S + bq x ,  acc = S . kk ,  S = a S      a = exp(g_t), bq = scale q_t, kk = k_t (vectors over the rows),  x = do_t[col]
template <int K>
__device__ void bwd_col_sweep(const BwdParams& P, BwdSmem& sm, int bh) {
    constexpr int NC = K / 2;
    const int tid = threadIdx.x, col = tid >> 1, part = tid & 1;
    const int b = bh / P.H, h = bh % P.H, T = P.T;
    const int64_t strideK = static_cast<int64_t>(P.H) * K, strideV = static_cast<int64_t>(P.H) * 64;
    const int64_t offK = (static_cast<int64_t>(b) * T * P.H + h) * K, offV = (static_cast<int64_t>(b) * T * P.H + h) * 64;
    const __half *pa = P.g + offK, *pq = P.q + offK, *pk = P.k + offK, *px = P.d_o + offV;
    __half* pout = P.dv + offV;

    float2 S[NC / 2];
#pragma unroll
    for (int j = 0; j < NC / 2; ++j) {
        const float* src = P.dht + (static_cast<int64_t>(bh) * K + part * NC + 2 * j) * 64 + col;
        S[j] = P.dht ? make_float2(src[0], src[64]) : make_float2(0.f, 0.f);
    }

    const int nchunks = (T + kBwdChunk - 1) / kBwdChunk;
    uint4 ra[K / 32], rq[K / 32], rk[K / 32], rx[2];
    auto fetch = [&](int ci) {
        const int t0 = (nchunks - 1 - ci) * kBwdChunk;
        bwd_fetch<K>(ra, pa, strideK, t0, T, tid);
        bwd_fetch<K>(rq, pq, strideK, t0, T, tid);
        bwd_fetch<K>(rk, pk, strideK, t0, T, tid);
        bwd_fetch<64>(rx, px, strideV, t0, T, tid);
    };
    if (nchunks > 0) fetch(0);
    for (int ci = 0; ci < nchunks; ++ci) {
        const int t0 = (nchunks - 1 - ci) * kBwdChunk;
        bwd_spread<K, true>(sm.tile[0], ra, 1.f, tid);
        bwd_spread<K, false>(sm.tile[1], rq, P.scale, tid);
        bwd_spread<K, false>(sm.tile[2], rk, 1.f, tid);
        bwd_spread<64, false>(sm.tile[3], rx, 1.f, tid);
        __syncthreads();
        if (ci + 1 < nchunks) fetch(ci + 1);
#pragma unroll 2
        for (int tt = 0; tt < kBwdChunk; ++tt) {
            const int t = kBwdChunk - 1 - tt;
            const float x = sm.tile[3][t * 64 + col];
            const float4* A = reinterpret_cast<const float4*>(&sm.tile[0][t * K + part * NC]);
            const float4* Q = reinterpret_cast<const float4*>(&sm.tile[1][t * K + part * NC]);
            const float4* Kk = reinterpret_cast<const float4*>(&sm.tile[2][t * K + part * NC]);
            const float2 xx = make_float2(x, x);
            float2 acc2 = make_float2(0.f, 0.f);
#pragma unroll
            for (int j = 0; j < NC / 4; ++j) {
                const float4 a = A[j], qq = Q[j], kk = Kk[j];
                S[2 * j] = bwd_fma2(make_float2(qq.x, qq.y), xx, S[2 * j]);
                S[2 * j + 1] = bwd_fma2(make_float2(qq.z, qq.w), xx, S[2 * j + 1]);
                acc2 = bwd_fma2(S[2 * j], make_float2(kk.x, kk.y), acc2);
                acc2 = bwd_fma2(S[2 * j + 1], make_float2(kk.z, kk.w), acc2);
                S[2 * j] = bwd_mul2(S[2 * j], make_float2(a.x, a.y));
                S[2 * j + 1] = bwd_mul2(S[2 * j + 1], make_float2(a.z, a.w));
            }
            float acc = acc2.x + acc2.y;
            acc += __shfl_xor_sync(0xffffffffu, acc, 1);
            if (part == 0) sm.out[t * 64 + col] = acc;
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
    const int bh = blockIdx.x, kind = blockIdx.y;
    if (kind == 0) bwd_row_sweep<K, 0>(P, sm, bh);
    else if (kind == 1) bwd_row_sweep<K, 1>(P, sm, bh);
    else bwd_col_sweep<K>(P, sm, bh);
}

// dg_t = sum_{s >= t} (q_s dq_s - k_s dk_s), per (batch, head, channel).  One CTA per (batch, head): 1024 / K slices
// of the sequence, each summed on its own first, then walked backwards from the total of the slices after it.
template <int K>
__global__ void __launch_bounds__(1024) gla_bwd_dg_kernel(const BwdParams P) {
    constexpr int kSlices = 1024 / K;
    __shared__ float total[kSlices][K];
    const int bh = blockIdx.x, b = bh / P.H, h = bh % P.H, T = P.T;
    const int c = threadIdx.x % K, s = threadIdx.x / K;
    const int64_t stride = static_cast<int64_t>(P.H) * K, off = (static_cast<int64_t>(b) * T * P.H + h) * K + c;
    const int per = (T + kSlices - 1) / kSlices, lo = s * per, hi = min(T, lo + per);
    const float last = P.g_last ? P.g_last[static_cast<int64_t>(bh) * K + c] : 0.f;
    float sum = 0.f;
    for (int t = lo; t < hi; ++t) sum += P.qdq[off + t * stride] - P.kdk[off + t * stride];
    if (lo < T && hi == T) sum += last;
    total[s][c] = sum;
    __syncthreads();
    float run = 0.f;
    for (int j = s + 1; j < kSlices; ++j) run += total[j][c];
    if (lo < T && hi == T) run += last;
    for (int t = hi - 1; t >= lo; --t) {
        run += P.qdq[off + t * stride] - P.kdk[off + t * stride];
        P.dg[off + t * stride] = run;
    }
}

}  // namespace gla
