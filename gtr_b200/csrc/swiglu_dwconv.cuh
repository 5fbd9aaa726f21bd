// Spatial SwiGLU middle step in one pass over memory:
//     out[b, r, c, :] = silu(gate[b, r, c, :]) * (bias + sum_{dr,dc in -1..1} w[dr, dc, :] * y[b, r+dr, c+dc, :])
// on tokens kept in their [B, L = hg*wg, C] layout (zero padding at the grid border).  Replaces, for the deploy
// form of the reference's SpatialSwiGLU (engine/gtr/backbone/vit_adapter_spatial_swiglu.py:50-60), the chain
// view/permute -> cuDNN depthwise 3x3 conv -> permute/reshape -> silu -> multiply and the layout copies around it.
//
// HBM-bound: gate and y are read once, out is written once (3 * 2 bytes per element).  What limits a direct form
// (every thread loading its 3x3 window from global memory: 3.4 loads of y per output, two thirds of them L2 hits)
// is the L2 -> SM path, which moved about 4 TB/s whatever the instruction mix; hence the shared-memory tile below.
#pragma once

#include <cuda_fp16.h>
#include <cstdint>

namespace gla {

__device__ __forceinline__ void dw_unpack8(const uint4& v, float* x) {
    const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 f = __half22float2(h[i]);
        x[2 * i] = f.x;
        x[2 * i + 1] = f.y;
    }
}

// acc[0..7] += w[0..7] * y[0..7] with the fp16 operands taken as they are: fma.rn.f32.f16 multiplies two fp16 values
// and accumulates in fp32 in one instruction (exact product, one rounding), so the taps cost no conversions.
__device__ __forceinline__ void dw_fma2(float& a0, float& a1, uint32_t w, uint32_t y) {
    asm("{\n\t.reg .b16 wl, wh, yl, yh;\n\t"
        "mov.b32 {wl, wh}, %2;\n\tmov.b32 {yl, yh}, %3;\n\t"
        "fma.rn.f32.f16 %0, wl, yl, %0;\n\tfma.rn.f32.f16 %1, wh, yh, %1;\n\t}"
        : "+f"(a0), "+f"(a1)
        : "r"(w), "r"(y));
}
__device__ __forceinline__ void dw_fma8(float* acc, const uint4& wv, const uint4& yv) {
    dw_fma2(acc[0], acc[1], wv.x, yv.x);
    dw_fma2(acc[2], acc[3], wv.y, yv.y);
    dw_fma2(acc[4], acc[5], wv.z, yv.z);
    dw_fma2(acc[6], acc[7], wv.w, yv.w);
}

// gate, y, out: [B, hg, wg, C] fp16 contiguous; wt: [3][3][C] fp16 (tap-major); bias: [C] fp16 or null.
// A CTA brings the y tile of kDwTileR x kDwTileC outputs plus its one-cell halo, for a slab of kDwSlab channel groups
// (8 channels each), into shared memory with cp.async -- every y element crosses the L2 -> SM path 1.4 times -- and
// each thread (one tile row, one channel group) then slides its 3x3 window of 16-byte vectors along the row out of
// shared memory.  The whole tile is in flight at once (45 KB per CTA, four CTAs per SM); consecutive threads hold
// consecutive channel groups, so every global access of a half-warp is 256 contiguous bytes.
#ifndef DW_TR
#define DW_TR 8
#endif
#ifndef DW_MINB
#define DW_MINB 4
#endif
#ifndef DW_TC
#define DW_TC 16
#endif
constexpr int kDwTileR = DW_TR, kDwTileC = DW_TC, kDwSlab = 16;
constexpr int kDwTileThreads = kDwTileR * kDwSlab;                                   // 128
constexpr int kDwTilePos = (kDwTileR + 2) * (kDwTileC + 2);                          // 180 positions
constexpr int kDwTileSmem = kDwTilePos * kDwSlab * 16;                               // 46,080 bytes

__device__ __forceinline__ void dw_cp_async16(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}

__global__ void __launch_bounds__(kDwTileThreads, DW_MINB) swiglu_dwconv_kernel(
    const __half* __restrict__ gate, const __half* __restrict__ y, const __half* __restrict__ wt,
    const __half* __restrict__ bias, __half* __restrict__ out, int B, int hg, int wg, int C) {
    extern __shared__ __align__(16) unsigned char dw_smem[];
    const int CG = C >> 3;
    const int nslab = (CG + kDwSlab - 1) / kDwSlab;
    const int tiles_c = (wg + kDwTileC - 1) / kDwTileC, tiles_r = (hg + kDwTileR - 1) / kDwTileR;
    // block -> (b, tile row, tile column, slab), slab fastest: neighbouring CTAs read neighbouring bytes
    long long rest = blockIdx.x;
    const int slab = static_cast<int>(rest % nslab); rest /= nslab;
    const int tc = static_cast<int>(rest % tiles_c); rest /= tiles_c;
    const int tr = static_cast<int>(rest % tiles_r);
    const int b = static_cast<int>(rest / tiles_r);
    const int r0 = tr * kDwTileR, c0 = tc * kDwTileC, cg0 = slab * kDwSlab;
    const int tid = threadIdx.x;
    const uint32_t sbase = static_cast<uint32_t>(__cvta_generic_to_shared(dw_smem));
    const uint4* y4 = reinterpret_cast<const uint4*>(y);
    const long long img = static_cast<long long>(b) * hg * wg;

    // ---- the gate vectors this thread will need (one tile row, 16 columns) are asked into L2 first: they are read
    // straight from global memory during the compute phase, two columns ahead of their use, which covers an L2 hit
    // but not a DRAM access under load.  One request per 128-byte line.
    {
        const int pci = tid % kDwSlab, prow = r0 + tid / kDwSlab, pcg = cg0 + pci;
        if ((pci & 7) == 0 && prow < hg && pcg < CG) {
            const uint4* gp = reinterpret_cast<const uint4*>(gate) + (img + static_cast<long long>(prow) * wg + c0) * CG + pcg;
            const int n = min(kDwTileC, wg - c0);
            for (int j = 0; j < n; ++j)
                asm volatile("prefetch.global.L2 [%0];" ::"l"(gp + static_cast<long long>(j) * CG) : "memory");
        }
    }

    // ---- fill: position (pr, pc) of the halo tile is grid cell (r0 - 1 + pr, c0 - 1 + pc); zeros outside the grid
    for (int idx = tid; idx < kDwTilePos * kDwSlab; idx += kDwTileThreads) {
        const int pos = idx / kDwSlab, ci = idx - pos * kDwSlab;
        const int pr = pos / (kDwTileC + 2), pc = pos - pr * (kDwTileC + 2);
        const int r = r0 - 1 + pr, c = c0 - 1 + pc, cg = cg0 + ci;
        const uint32_t dst = sbase + static_cast<uint32_t>(idx) * 16u;
        if (r >= 0 && r < hg && c >= 0 && c < wg && cg < CG)
            dw_cp_async16(dst, y4 + (img + static_cast<long long>(r) * wg + c) * CG + cg);
        else
            asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(dst), "r"(0u) : "memory");
    }
    asm volatile("cp.async.commit_group;" ::: "memory");

    // ---- this thread: tile row trow, channel group cg; weights and bias while the tile is in flight
    const int ci = tid % kDwSlab, trow = tid / kDwSlab;
    const int cg = cg0 + ci, r = r0 + trow;
    const bool active = cg < CG && r < hg;
    const int cgc = cg < CG ? cg : CG - 1;
    uint4 wv[9];
#pragma unroll
    for (int k = 0; k < 9; ++k) wv[k] = __ldg(reinterpret_cast<const uint4*>(wt) + static_cast<long long>(k) * CG + cgc);
    float bv[8];
    if (bias != nullptr) dw_unpack8(__ldg(reinterpret_cast<const uint4*>(bias) + cgc), bv);
    else {
#pragma unroll
        for (int i = 0; i < 8; ++i) bv[i] = 0.f;
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();
    if (!active) return;

    auto ld = [&](int pr, int pc) {
        uint4 v;
        const uint32_t a = sbase + static_cast<uint32_t>((pr * (kDwTileC + 2) + pc) * kDwSlab + ci) * 16u;
        asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
        return v;
    };
    const long long base = (img + static_cast<long long>(r) * wg) * CG + cg;
    const uint4* g4 = reinterpret_cast<const uint4*>(gate);
    uint4* o4 = reinterpret_cast<uint4*>(out);
    const int ncol = min(kDwTileC, wg - c0);
    // the 3x3 window slides along the row: three columns of three 16-byte vectors in registers; the column loop is
    // unrolled so that the columns change roles by renaming, not by moves
    uint4 win[3][3];                     // win[column slot][row]
#pragma unroll
    for (int rr = 0; rr < 3; ++rr) { win[0][rr] = ld(trow + rr, 0); win[1][rr] = ld(trow + rr, 1); }
    // the gate vectors come straight from global memory (L2 after the prefetch above), two columns ahead of their use
    const long long pcol = base + static_cast<long long>(c0) * CG;
    uint4 gq[3];
    gq[0] = __ldg(g4 + pcol);
    gq[1] = ncol > 1 ? __ldg(g4 + pcol + CG) : gq[0];
#pragma unroll
    for (int j = 0; j < kDwTileC; ++j) {
        if (j < ncol) {
            const int sl = j % 3, sm = (j + 1) % 3, sn = (j + 2) % 3;     // left, middle, new column slots
#pragma unroll
            for (int rr = 0; rr < 3; ++rr) win[sn][rr] = ld(trow + rr, j + 2);
            const long long p = pcol + static_cast<long long>(j) * CG;
            if (j + 2 < ncol) gq[(j + 2) % 3] = __ldg(g4 + p + 2 * static_cast<long long>(CG));
            float acc[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[i] = bv[i];
#pragma unroll
            for (int rr = 0; rr < 3; ++rr) {
                dw_fma8(acc, wv[3 * rr + 0], win[sl][rr]);
                dw_fma8(acc, wv[3 * rr + 1], win[sm][rr]);
                dw_fma8(acc, wv[3 * rr + 2], win[sn][rr]);
            }
            float g[8];
            dw_unpack8(gq[j % 3], g);
            uint4 o;
            __half2* oh = reinterpret_cast<__half2*>(&o);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float h0 = 0.5f * g[2 * i], h1 = 0.5f * g[2 * i + 1];      // silu(x) = h + h * tanh(h), h = x / 2
                float t0, t1;
                asm("tanh.approx.f32 %0, %1;" : "=f"(t0) : "f"(h0));
                asm("tanh.approx.f32 %0, %1;" : "=f"(t1) : "f"(h1));
                oh[i] = __floats2half2_rn(fmaf(h0, t0, h0) * acc[2 * i], fmaf(h1, t1, h1) * acc[2 * i + 1]);
            }
            o4[p] = o;
        }
    }
}

}  // namespace gla

namespace gla {

// LayerNorm over rows of D fp16 values (D a multiple of 8, D <= 2048), affine, fp32 statistics: one warp per row,
// the row held in registers between the mean, the variance and the output pass, so that x is read once and y written
// once (the backbone's norms run at a quarter of that with the framework's kernel).
// kVec = 16-byte vectors per lane, chosen by the host from D: a narrow row must not pay for the registers of the
// widest one (occupancy is what keeps enough loads in flight here).
constexpr int kLnMaxVec = 8;

// y may alias x (in-place use): x is read with plain loads and neither pointer is declared restrict.
template <int kVec>
__global__ void __launch_bounds__(256) layernorm_rows_kernel(const __half* x, const __half* __restrict__ w,
                                                             const __half* __restrict__ b, __half* y,
                                                             long long rows, int D, float eps) {
    const long long row = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (row >= rows) return;
    const int nvec = D >> 3;
    const uint4* x4 = reinterpret_cast<const uint4*>(x) + row * nvec;
    float v[kVec][8];
    float sum = 0.f;
#pragma unroll
    for (int k = 0; k < kVec; ++k) {
        const int i = lane + 32 * k;
        if (i < nvec) {
            dw_unpack8(x4[i], v[k]);
#pragma unroll
            for (int e = 0; e < 8; ++e) sum += v[k][e];
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    const float mean = sum / static_cast<float>(D);
    float sq = 0.f;
#pragma unroll
    for (int k = 0; k < kVec; ++k) {
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
    for (int k = 0; k < kVec; ++k) {
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
