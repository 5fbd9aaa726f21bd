// Spatial SwiGLU middle step in one pass over memory:
//     out[b, r, c, :] = silu(gate[b, r, c, :]) * (bias + sum_{dr,dc in -1..1} w[dr, dc, :] * y[b, r+dr, c+dc, :])
// on tokens kept in their [B, L = hg*wg, C] layout (zero padding at the grid border).  Replaces, for the deploy
// form of the reference's SpatialSwiGLU (engine/gtr/backbone/vit_adapter_spatial_swiglu.py:50-60), the chain
// view/permute -> cuDNN depthwise 3x3 conv -> permute/reshape -> silu -> multiply and the layout copies around it.
//
// HBM-bound: gate and y are read once, out is written once (3 * 2 bytes per element); the 3x3 window makes every
// y element be loaded three times, twice from L2.  A thread owns 8 channels (one 16-byte vector) and a strip of
// kStrip consecutive grid columns of one grid row; it slides a 3x3 window of vectors along the strip, so each step
// loads three new vectors (rows r-1, r, r+1 of the next column), one gate vector, and stores one output vector.
// Consecutive threads hold consecutive channel groups: every access of a warp is 512 contiguous bytes.
#pragma once

#include <cuda_fp16.h>
#include <cstdint>

namespace gla {

constexpr int kDwStrip = 16;

__device__ __forceinline__ void dw_unpack8(const uint4& v, float* x) {
    const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 f = __half22float2(h[i]);
        x[2 * i] = f.x;
        x[2 * i + 1] = f.y;
    }
}

__device__ __forceinline__ void dw_fma8(float* acc, const uint4& wv, const uint4& yv) {
    float w[8], y[8];
    dw_unpack8(wv, w);
    dw_unpack8(yv, y);
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = fmaf(w[i], y[i], acc[i]);
}

// gate, y, out: [B, hg, wg, C] fp16 contiguous; wt: [3][3][C] fp16 (tap-major); bias: [C] fp16 or null.
__global__ void __launch_bounds__(128, 4) swiglu_dwconv_kernel(const __half* __restrict__ gate, const __half* __restrict__ y,
                                                            const __half* __restrict__ wt, const __half* __restrict__ bias,
                                                            __half* __restrict__ out, int B, int hg, int wg, int C) {
    const int CG = C >> 3;
    const int nstrips = (wg + kDwStrip - 1) / kDwStrip;
    const long long total = static_cast<long long>(B) * hg * nstrips * CG;
    const long long t = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (t >= total) return;
    const int cg = static_cast<int>(t % CG);
    long long rest = t / CG;
    const int s = static_cast<int>(rest % nstrips);
    rest /= nstrips;
    const int r = static_cast<int>(rest % hg);
    const int b = static_cast<int>(rest / hg);
    const int c0 = s * kDwStrip, c1 = min(c0 + kDwStrip, wg);

    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
    const uint4* w4 = reinterpret_cast<const uint4*>(wt) + cg;          // + tap * CG
    uint4 wv[9];
#pragma unroll
    for (int k = 0; k < 9; ++k) wv[k] = __ldg(w4 + static_cast<long long>(k) * CG);
    float bv[8];
    if (bias != nullptr) dw_unpack8(__ldg(reinterpret_cast<const uint4*>(bias) + cg), bv);
    else {
#pragma unroll
        for (int i = 0; i < 8; ++i) bv[i] = 0.f;
    }

    // vector index of (b, row, col): ((b * hg + row) * wg + col) * CG + cg
    const long long row_stride = static_cast<long long>(wg) * CG;
    const long long base = (static_cast<long long>(b) * hg + r) * row_stride + cg;
    const uint4* y4 = reinterpret_cast<const uint4*>(y);
    const bool up = r > 0, down = r + 1 < hg;
    auto load_col = [&](int c, uint4& a, uint4& m, uint4& d) {
        if (c < 0 || c >= wg) {
            a = m = d = zero;
            return;
        }
        const long long p = base + static_cast<long long>(c) * CG;
        a = up ? __ldg(y4 + p - row_stride) : zero;
        m = __ldg(y4 + p);
        d = down ? __ldg(y4 + p + row_stride) : zero;
    };
    uint4 l0, l1, l2, m0, m1, m2, n0, n1, n2;     // window columns c-1 (l), c (m), c+1 (n); rows r-1, r, r+1
    load_col(c0 - 1, l0, l1, l2);
    load_col(c0, m0, m1, m2);
    for (int c = c0; c < c1; ++c) {
        load_col(c + 1, n0, n1, n2);
        const long long p = base + static_cast<long long>(c) * CG;
        const uint4 gv = __ldg(reinterpret_cast<const uint4*>(gate) + p);
        float acc[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] = bv[i];
        dw_fma8(acc, wv[0], l0); dw_fma8(acc, wv[1], m0); dw_fma8(acc, wv[2], n0);
        dw_fma8(acc, wv[3], l1); dw_fma8(acc, wv[4], m1); dw_fma8(acc, wv[5], n1);
        dw_fma8(acc, wv[6], l2); dw_fma8(acc, wv[7], m2); dw_fma8(acc, wv[8], n2);
        float g[8];
        dw_unpack8(gv, g);
        uint4 o;
        __half2* oh = reinterpret_cast<__half2*>(&o);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            // silu(x) = h + h * tanh(h), h = x / 2
            const float h0 = 0.5f * g[2 * i], h1 = 0.5f * g[2 * i + 1];
            float t0, t1;
            asm("tanh.approx.f32 %0, %1;" : "=f"(t0) : "f"(h0));
            asm("tanh.approx.f32 %0, %1;" : "=f"(t1) : "f"(h1));
            oh[i] = __floats2half2_rn(fmaf(h0, t0, h0) * acc[2 * i], fmaf(h1, t1, h1) * acc[2 * i + 1]);
        }
        reinterpret_cast<uint4*>(out)[p] = o;
        l0 = m0; l1 = m1; l2 = m2;
        m0 = n0; m1 = n1; m2 = n2;
    }
}

}  // namespace gla

namespace gla {

// LayerNorm over rows of D fp16 values (D a multiple of 8, D <= 2048), affine, fp32 statistics: one warp per row,
// the row held in registers between the mean, the variance and the output pass, so that x is read once and y written
// once (the backbone's norms run at a quarter of that with the framework's kernel).
constexpr int kLnMaxVec = 8;      // 16-byte vectors per lane

__global__ void __launch_bounds__(256) layernorm_rows_kernel(const __half* __restrict__ x, const __half* __restrict__ w,
                                                             const __half* __restrict__ b, __half* __restrict__ y,
                                                             long long rows, int D, float eps) {
    const long long row = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (row >= rows) return;
    const int nvec = D >> 3;
    const uint4* x4 = reinterpret_cast<const uint4*>(x) + row * nvec;
    float v[kLnMaxVec][8];
    float sum = 0.f;
#pragma unroll
    for (int k = 0; k < kLnMaxVec; ++k) {
        const int i = lane + 32 * k;
        if (i < nvec) {
            dw_unpack8(__ldg(x4 + i), v[k]);
#pragma unroll
            for (int e = 0; e < 8; ++e) sum += v[k][e];
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    const float mean = sum / static_cast<float>(D);
    float sq = 0.f;
#pragma unroll
    for (int k = 0; k < kLnMaxVec; ++k) {
        if (lane + 32 * k < nvec) {
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                const float d = v[k][e] - mean;
                sq = fmaf(d, d, sq);
            }
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
    const float rstd = rsqrtf(sq / static_cast<float>(D) + eps);
    uint4* y4 = reinterpret_cast<uint4*>(y) + row * nvec;
#pragma unroll
    for (int k = 0; k < kLnMaxVec; ++k) {
        const int i = lane + 32 * k;
        if (i < nvec) {
            float wv[8], bv[8];
            dw_unpack8(__ldg(reinterpret_cast<const uint4*>(w) + i), wv);
            if (b != nullptr) dw_unpack8(__ldg(reinterpret_cast<const uint4*>(b) + i), bv);
            uint4 o;
            __half2* oh = reinterpret_cast<__half2*>(&o);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float a0 = (v[k][2 * e] - mean) * rstd * wv[2 * e] + (b != nullptr ? bv[2 * e] : 0.f);
                const float a1 = (v[k][2 * e + 1] - mean) * rstd * wv[2 * e + 1] + (b != nullptr ? bv[2 * e + 1] : 0.f);
                oh[e] = __floats2half2_rn(a0, a1);
            }
            y4[i] = o;
        }
    }
}

}  // namespace gla
