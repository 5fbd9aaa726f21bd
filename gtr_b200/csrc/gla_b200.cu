// Host side of libgla_b200.so: argument checks, tensor-map construction, workspace layout
// and launches behind the C ABI declared in include/gla_b200.h.  No allocation, no
// synchronisation on the forward path.
#include "gla_b200.h"

#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <vector>

#include "gla_kernel.cuh"
#include "swiglu_dwconv.cuh"
#include "gla_bwd.cuh"

namespace {

thread_local char g_cuda_err[256] = "";

void note_cuda(const char* what, cudaError_t e) {
    snprintf(g_cuda_err, sizeof(g_cuda_err), "%s: %s", what, cudaGetErrorString(e));
}
void note_cu(const char* what, int e) { snprintf(g_cuda_err, sizeof(g_cuda_err), "%s: CUresult %d", what, e); }

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled() {
    static EncodeTiledFn fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            p = nullptr;
        return reinterpret_cast<EncodeTiledFn>(p);
    }();
    return fn;
}

// The forward kernel's instantiations: bit 2 fused epilogue, bit 1 raw-logit gates, bit 0 reversed scan.
const void* fwd_kernel(int variant) {
    using gla::gla_fwd_kernel;
    static const void* const table[8] = {
        reinterpret_cast<const void*>(&gla_fwd_kernel<false, false, false>), reinterpret_cast<const void*>(&gla_fwd_kernel<false, false, true>),
        reinterpret_cast<const void*>(&gla_fwd_kernel<false, true, false>),  reinterpret_cast<const void*>(&gla_fwd_kernel<false, true, true>),
        reinterpret_cast<const void*>(&gla_fwd_kernel<true, false, false>),  reinterpret_cast<const void*>(&gla_fwd_kernel<true, false, true>),
        reinterpret_cast<const void*>(&gla_fwd_kernel<true, true, false>),   reinterpret_cast<const void*>(&gla_fwd_kernel<true, true, true>)};
    return table[variant & 7];
}

struct DeviceInfo {
    bool ok = false;
    int sms = 0;
    bool attr_set = false;
};
std::mutex g_mu;
DeviceInfo g_dev[64];

int device_info(int dev, DeviceInfo* out) {
    std::lock_guard<std::mutex> lock(g_mu);
    DeviceInfo& d = g_dev[dev];
    if (!d.attr_set) {
        int major = 0, sms = 0;
        cudaError_t e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
        if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        if (e != cudaSuccess) { note_cuda("cudaDeviceGetAttribute", e); return GLA_B200_ERR_CUDA; }
        if (major != 10) {
            snprintf(g_cuda_err, sizeof(g_cuda_err), "device %d has compute capability %d.x, need 10.x", dev, major);
            return GLA_B200_ERR_DEVICE;
        }
        for (int v = 0; v < 8 && e == cudaSuccess; ++v)
            e = cudaFuncSetAttribute(fwd_kernel(v), cudaFuncAttributeMaxDynamicSharedMemorySize, gla::kSmemBytes);
        if (e != cudaSuccess) { note_cuda("cudaFuncSetAttribute", e); return GLA_B200_ERR_CUDA; }
        // The warpgroups of the kernel re-divide the registers the CTA was launched with (setmaxnreg); a group that
        // asks for more than the others release would wait for ever, so the budgets are checked against what this
        // build of the kernel really gets at launch.
        cudaFuncAttributes fa;
        e = cudaFuncGetAttributes(&fa, fwd_kernel(0));
        if (e != cudaSuccess) { note_cuda("cudaFuncGetAttributes", e); return GLA_B200_ERR_CUDA; }
        if (fa.numRegs * gla::kThreads < gla::kRegBudgetTotal) {
            snprintf(g_cuda_err, sizeof(g_cuda_err), "kernel launches with %d registers per thread, its register budgets need %d",
                     fa.numRegs, (gla::kRegBudgetTotal + gla::kThreads - 1) / gla::kThreads);
            return GLA_B200_ERR_DEVICE;
        }
        d.ok = true;
        d.sms = sms;
        d.attr_set = true;
    }
    *out = d;
    return GLA_B200_OK;
}

// ---- workspace layout ------------------------------------------------------------------
struct WsLayout {
    size_t ctrl, flags, agg, incl, total;
    size_t clear_bytes;   // ctrl + flags, zeroed before every launch
};

size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

WsLayout ws_layout(size_t nseq, size_t ns) {
    WsLayout L;
    L.ctrl = 0;
    L.flags = 256;
    L.clear_bytes = 256 + align_up(nseq * ns * 4, 256);
    // segment aggregates and inclusive states are exchanged between the work items of one sequence only:
    // unsegmented sequences (ns == 1) need none, whatever their number
    const size_t slots = ns > 1 ? nseq * ns : 0;
    L.agg = L.clear_bytes;
    L.incl = L.agg + align_up(slots * gla::kAggStride * 4, 256);
    L.total = L.incl + align_up(slots * gla::kD * gla::kD * 4, 256);
    return L;
}

constexpr int kMinAutoCps = 4;   // smallest automatic segment length; also sizes the advertised workspace

int num_chunks(int T) { return (T + gla::kChunk - 1) / gla::kChunk; }

// Segment length that minimises a simple cost model of the persistent kernel: the work items
// (sequences x segments) run in rounds of `slots` CTAs; an item costs its chunks once for the
// output pass plus about half of that for the state-only pre-pass every segment but the last
// needs.  One segment per sequence avoids the pre-pass but leaves slots idle when there are few
// sequences; many segments fill the machine but pay the pre-pass and round up to whole rounds.
int auto_chunks_per_segment(int NT, int nseq, int slots, size_t workspace_bytes) {
    int best_cps = NT;
    double best = 1e300;
    for (int cps = NT; cps >= 1; --cps) {
        const int ns = (NT + cps - 1) / cps;
        if (ns > 1 && cps < kMinAutoCps) break;
        if (cps != (NT + ns - 1) / ns) continue;               // only the balanced split for each segment count
        // a split whose scratch does not fit the caller's workspace is not a candidate: the policy then settles
        // for a coarser one (one segment per sequence needs next to nothing)
        if (ns > 1 && ws_layout(static_cast<size_t>(nseq), static_cast<size_t>(ns)).total > workspace_bytes) continue;
        const long items = static_cast<long>(nseq) * ns;
        const long rounds = (items + slots - 1) / slots;
        const double per_item = cps * (1.0 + (ns > 1 ? 0.5 * (ns - 1) / ns : 0.0)) + (ns > 1 ? 1.0 : 0.0);
        const double cost = rounds * per_item;
        if (cost < best - 1e-9) { best = cost; best_cps = cps; }
    }
    return best_cps;
}

// Staggered plan for r = slots / nseq CTAs per sequence, 2 <= r < kMaxPlanSegments (gla::Params::plan): segment 0 of
// `pre` x the length of the others, r equal ones after it.  `pre` is what a pre-pass chunk costs next to an output-pass
// chunk while both kinds run side by side; measured on 100 chunks with three CTAs per sequence, the fastest splits are
// 18 + 28 + 27 + 27 for the plain operator (and with raw gate logits, which cost both passes) and 14 + 29 + 29 + 28 with
// the fused epilogue (which costs the output pass only).  In units of one chunk's output pass every CTA then works
// (1 + pre) x the middle segments' length.  Returns that cost (plus one for the look-back), or a negative number when
// the plan does not apply.
constexpr double kPlanPrePassPlain = 0.68, kPlanPrePassGated = 0.48;
double staggered_plan(int NT, int nseq, int slots, size_t workspace_bytes, double pre, int* seg_start, int* ns_out) {
    const int r = nseq > 0 ? slots / nseq : 0;
    if (r < 2 || r + 1 > gla::kMaxPlanSegments || NT < kMinAutoCps * (r + 1)) return -1.0;
    if (ws_layout(static_cast<size_t>(nseq), static_cast<size_t>(r + 1)).total > workspace_bytes) return -1.0;
    const double mid = NT / (r + pre);
    int n0 = static_cast<int>(pre * mid + 0.5);
    if (n0 < 1) n0 = 1;
    const int rest = NT - n0;
    seg_start[0] = 0;
    seg_start[1] = n0;
    for (int i = 0; i < r; ++i) seg_start[i + 2] = seg_start[i + 1] + rest / r + (i < rest % r ? 1 : 0);
    *ns_out = r + 1;
    const int longest = rest / r + (rest % r ? 1 : 0);
    const double with_pass = (1.0 + pre) * longest, relay = n0 + (seg_start[r + 1] - seg_start[r]);
    return (with_pass > relay ? with_pass : relay) + 1.0;
}

// Relay plan (gla::Params::plan == 2) for more sequences than CTAs: the number of equal segments, without pre-passes,
// that minimises rounds x (segment length + one chunk's worth of look-back); 1 when whole sequences are as good.
int relay_segments(int NT, int nseq, int slots, size_t workspace_bytes, double* cost_out) {
    int best = 1;
    double best_cost = static_cast<double>((nseq + slots - 1) / slots) * NT;
    for (int ns = 2; ns <= 8; ++ns) {
        const int cps = (NT + ns - 1) / ns;
        if (cps < kMinAutoCps || (NT + cps - 1) / cps != ns) continue;
        if (ws_layout(static_cast<size_t>(nseq), static_cast<size_t>(ns)).total > workspace_bytes) continue;
        const long rounds = (static_cast<long>(nseq) * ns + slots - 1) / slots;
        const double cost = rounds * (cps + 1.0);
        if (cost < best_cost * 0.97) { best_cost = cost; best = ns; }       // only for a gain worth the extra state traffic
    }
    *cost_out = best_cost;
    return best;
}

// ---- tensor maps ------------------------------------------------------------------------
struct MapKey {
    const void* ptr[gla::kNumTensors];
    int64_t stride[gla::kNumTensors][3];
    int B, T, H, K, Hc, Wc, col;
    int dev;
    bool operator==(const MapKey& o) const { return memcmp(this, &o, sizeof(MapKey)) == 0; }
};
struct MapEntry {
    MapKey key;
    gla::Maps maps;
};
std::vector<MapEntry> g_map_cache;
constexpr size_t kMapCacheMax = 64;

int build_maps(const MapKey& key, gla::Maps* out) {
    EncodeTiledFn enc = encode_tiled();
    if (!enc) {
        snprintf(g_cuda_err, sizeof(g_cuda_err), "cuTensorMapEncodeTiled is not available from this driver");
        return GLA_B200_ERR_DEVICE;
    }
    for (int t = 0; t < gla::kNumTensors; ++t) {
        if (key.ptr[t] == nullptr) continue;
        const int64_t sb = key.stride[t][0], st = key.stride[t][1], sh = key.stride[t][2];
        // dims: (d, head, row-in-column, column, batch)
        // q, k and g of a K = 32 head: the channel dimension keeps its true extent while the box stays 64 wide, so
        // channels 32..63 of every tile are filled with zeros by the copy engine (out-of-bounds fill)
        const bool key_side = t == gla::TQ || t == gla::TK || t == gla::TG;
        const cuuint64_t gdim[5] = {static_cast<cuuint64_t>(key_side ? key.K : gla::kD), static_cast<cuuint64_t>(key.H),
                                    static_cast<cuuint64_t>(key.Hc), static_cast<cuuint64_t>(key.Wc),
                                    static_cast<cuuint64_t>(key.B)};
        const int64_t row_stride = key.col ? st * key.Wc : st;
        const int64_t col_stride = key.col ? st : st * key.T;
        const cuuint64_t gstr[4] = {static_cast<cuuint64_t>(sh) * 2, static_cast<cuuint64_t>(row_stride) * 2,
                                    static_cast<cuuint64_t>(col_stride) * 2, static_cast<cuuint64_t>(sb) * 2};
        const cuuint32_t estr[5] = {1, 1, 1, 1, 1};
        for (int b = 0; b < gla::kNumBoxes; ++b) {
            const cuuint32_t box[5] = {static_cast<cuuint32_t>(gla::kD), 1, static_cast<cuuint32_t>(64 >> (2 * b)), 1, 1};
            CUresult r = enc(&out->m[t][b], CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 5, const_cast<void*>(key.ptr[t]), gdim,
                             gstr, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                             CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
            if (r != CUDA_SUCCESS) { note_cu("cuTensorMapEncodeTiled", static_cast<int>(r)); return GLA_B200_ERR_CUDA; }
        }
    }
    return GLA_B200_OK;
}

int get_maps(const MapKey& key, gla::Maps* out) {
    {
        std::lock_guard<std::mutex> lock(g_mu);
        for (const MapEntry& e : g_map_cache)
            if (e.key == key) { *out = e.maps; return GLA_B200_OK; }
    }
    MapEntry e;
    memset(&e, 0, sizeof(e));
    e.key = key;
    int rc = build_maps(key, &e.maps);
    if (rc != GLA_B200_OK) return rc;
    *out = e.maps;
    std::lock_guard<std::mutex> lock(g_mu);
    if (g_map_cache.size() >= kMapCacheMax) g_map_cache.erase(g_map_cache.begin());
    g_map_cache.push_back(e);
    return GLA_B200_OK;
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

int resolve_strides(const int64_t in[3], int T, int H, int D, int64_t out[3]) {
    if (in[0] == 0 && in[1] == 0 && in[2] == 0) {
        out[0] = static_cast<int64_t>(T) * H * D;
        out[1] = static_cast<int64_t>(H) * D;
        out[2] = D;
        return GLA_B200_OK;
    }
    for (int i = 0; i < 3; ++i) {
        if (in[i] <= 0) return GLA_B200_ERR_ARG;
        if (in[i] % 8 != 0) return GLA_B200_ERR_ALIGN;
        out[i] = in[i];
    }
    if (out[2] < D) return GLA_B200_ERR_ARG;
    return GLA_B200_OK;
}

// ---- standalone RMSNorm * w * silu(gate), rows of 64 fp16 --------------------------------
// y may alias x (in-place use): x is read with plain loads and neither pointer is declared restrict.
__global__ void __launch_bounds__(256) rmsnorm_gated_kernel(const __half* x, const __half* __restrict__ g,
                                                            const __half* __restrict__ wgt, __half* y,
                                                            int64_t rows, float eps) {
    // 8 lanes per row, 8 fp16 (16 bytes) per lane; a warp covers 4 consecutive rows = 512 contiguous bytes
    const int64_t row = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 3;
    const int sub = threadIdx.x & 7;
    const bool live = row < rows;
    float xv[8], gv[8], wv[8];
    uint4 xr = make_uint4(0, 0, 0, 0), gr = xr;
    const uint4 wr = __ldg(reinterpret_cast<const uint4*>(wgt) + sub);
    if (live) {
        xr = *(reinterpret_cast<const uint4*>(x + row * 64) + sub);
        gr = __ldg(reinterpret_cast<const uint4*>(g + row * 64) + sub);
    }
    const uint32_t* xp = &xr.x;
    const uint32_t* gp = &gr.x;
    const uint32_t* wp = &wr.x;
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 a = gla::unpack_half2(xp[i]), b = gla::unpack_half2(gp[i]), c = gla::unpack_half2(wp[i]);
        xv[2 * i] = a.x; xv[2 * i + 1] = a.y;
        gv[2 * i] = b.x; gv[2 * i + 1] = b.y;
        wv[2 * i] = c.x; wv[2 * i + 1] = c.y;
        ss += a.x * a.x + a.y * a.y;
    }
    ss += __shfl_xor_sync(0xffffffffu, ss, 1);
    ss += __shfl_xor_sync(0xffffffffu, ss, 2);
    ss += __shfl_xor_sync(0xffffffffu, ss, 4);
    const float r = rsqrtf(ss * (1.f / 64.f) + eps);
    uint32_t o[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float y0 = xv[2 * i] * r * wv[2 * i] * (gv[2 * i] / (1.f + __expf(-gv[2 * i])));
        const float y1 = xv[2 * i + 1] * r * wv[2 * i + 1] * (gv[2 * i + 1] / (1.f + __expf(-gv[2 * i + 1])));
        o[i] = gla::pack_half2_sat(y0, y1);
    }
    if (live) *(reinterpret_cast<uint4*>(y + row * 64) + sub) = make_uint4(o[0], o[1], o[2], o[3]);
}


// ---- streaming probe: the loading scheme of the forward kernel with nothing behind it ---------------------
constexpr int kProbeStages = 5, kProbeThreads = 64;
__device__ __forceinline__ bool probe_wait(uint32_t bar, uint32_t parity) {
    for (int n = 0; n < (1 << 22); ++n)
        if (gla::mbar_try_wait(bar, parity)) return true;
    return false;                                    // bounded: give up and say so
}
__global__ void __launch_bounds__(kProbeThreads) stream_probe_kernel(const __grid_constant__ CUtensorMap map, int heads, int tiles,
                                                                     int chunks, int slab_rows, int* status) {
    extern __shared__ uint8_t probe_smem[];
    const uint32_t sb = (gla::smem_u32(probe_smem) + 1023u) & ~1023u;
    __shared__ uint64_t full[kProbeStages], empty[kProbeStages];
    const int tid = threadIdx.x;
    if (tid == 0) {
        for (int s = 0; s < kProbeStages; ++s) { gla::mbar_init(gla::smem_u32(&full[s]), 1); gla::mbar_init(gla::smem_u32(&empty[s]), 1); }
        gla::fence_mbar_init();
    }
    __syncthreads();
    const int head = blockIdx.x % heads, region = blockIdx.x / heads;
    if (tid == 32) {                                 // consumer: hands every stage back as soon as it has landed
        for (int i = 0; i < chunks; ++i) {
            const int s = i % kProbeStages;
            if (!probe_wait(gla::smem_u32(&full[s]), (i / kProbeStages) & 1)) { if (status) atomicExch(status, 1); break; }
            gla::mbar_arrive(gla::smem_u32(&empty[s]));
        }
    } else if (tid == 0) {                           // producer
        for (int i = 0; i < chunks; ++i) {
            const int s = i % kProbeStages;
            if (i >= kProbeStages && !probe_wait(gla::smem_u32(&empty[s]), ((i / kProbeStages) & 1) ^ 1)) { if (status) atomicExch(status, 2); break; }
            const uint32_t bar = gla::smem_u32(&full[s]);
            gla::mbar_arrive_expect_tx(bar, static_cast<uint32_t>(tiles) * gla::kTileBytes);
            const int row = (region * chunks + i) * gla::kChunk;
            for (int t = 0; t < tiles; ++t)
                asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
                             ::"r"(sb + static_cast<uint32_t>(s * 4 + t) * gla::kTileBytes), "l"(reinterpret_cast<uint64_t>(&map)), "r"(bar),
                               "r"(0), "r"(head), "r"(t * slab_rows + row) : "memory");
        }
    }
    __syncthreads();
}

}  // namespace

// ---------------------------------------------------------------------------------------------
// Scratch for gla_b200_forward_static: forward without any caller-provided or allocated scratch.
//
// For hosts that must not touch the device allocator when they call the operator: an inference
// server that handed all device memory to its own pool at start-up (a cudaMalloc there fails or
// stalls every stream of the process), a plugin whose framework gives it no workspace, or a
// real-time loop whose memory budget was fixed before it started.  The kernel's scratch (ticket,
// status word, per-segment flags, segment aggregates and inclusive states) then lives in the array
// below, which every GPU that loads this library holds until the process exits.
//
// In host code the array's name is only a handle, not a device address, so the address is looked
// up with cudaGetSymbolAddress, once per device and with that device current.  That happens in the
// first call on a device: make that call before any stream capture.
// All calls share the one array per device; it keeps the previous call's contents.  The words that
// must start at zero (ticket, status, flags) are cleared on the stream at the start of every call;
// everything else is written before it is read.  Two calls that overlap on the same GPU (different
// streams, or graph branches) would race on the array: serialise them.
static __device__ __align__(256) unsigned char g_static_scratch[GLA_B200_STATIC_SCRATCH_BYTES];

namespace {
std::mutex g_static_mu;
void* g_static_ptr[64] = {nullptr};

// Device address of the built-in array on the current device (looked up on first use).
int static_scratch(void** out) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) { note_cuda("cudaGetDevice", e); return GLA_B200_ERR_CUDA; }
    if (dev < 0 || dev >= 64) return GLA_B200_ERR_DEVICE;
    std::lock_guard<std::mutex> lock(g_static_mu);
    if (g_static_ptr[dev] == nullptr) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_static_scratch);      // address on the current device
        if (e != cudaSuccess || p == nullptr) { note_cuda("cudaGetSymbolAddress", e); return GLA_B200_ERR_CUDA; }
        g_static_ptr[dev] = p;
    }
    *out = g_static_ptr[dev];
    return GLA_B200_OK;
}
}  // namespace

extern "C" {

int gla_b200_version(void) { return GLA_B200_VERSION; }

const char* gla_b200_strerror(int code) {
    switch (code) {
        case GLA_B200_OK: return "ok";
        case GLA_B200_ERR_NULL: return "a required pointer is NULL";
        case GLA_B200_ERR_SHAPE: return "unsupported shape (need K = 32 or 64, V = 64, B,T,H >= 0, grid_h*grid_w == T)";
        case GLA_B200_ERR_ALIGN: return "pointer or stride is not 16-byte aligned";
        case GLA_B200_ERR_DIRECTION: return "direction must be 0 (row), 1 (row reversed), 2 (column) or 3 (column reversed)";
        case GLA_B200_ERR_WORKSPACE: return "workspace is NULL, misaligned or smaller than gla_b200_workspace_bytes()";
        case GLA_B200_ERR_DEVICE: return "the current device is not an sm_100 GPU or the driver lacks tensor-map support";
        case GLA_B200_ERR_CUDA: return "a CUDA call failed (see gla_b200_last_cuda_error)";
        case GLA_B200_ERR_TIMEOUT: return "a bounded wait inside the kernel expired; outputs are undefined";
        case GLA_B200_ERR_ARG: return "invalid argument";
        case GLA_B200_ERR_STATIC_SCRATCH:
            return "the problem needs more scratch than the library's built-in array (GLA_B200_STATIC_SCRATCH_BYTES); "
                   "use gla_b200_forward with a caller-owned workspace";
        default: return "unknown gla_b200 error code";
    }
}

const char* gla_b200_last_cuda_error(void) { return g_cuda_err; }

size_t gla_b200_workspace_bytes(int32_t B, int32_t T, int32_t H, int32_t K, int32_t V) {
    if (B < 0 || T < 0 || H < 0 || (K != 32 && K != gla::kD) || V != gla::kD) return 0;
    const size_t nseq = static_cast<size_t>(B) * H;
    const size_t ns = static_cast<size_t>((num_chunks(T) + kMinAutoCps - 1) / kMinAutoCps);
    return ws_layout(nseq, ns ? ns : 1).total;
}

int gla_b200_forward(const gla_b200_args* a, void* stream_v) {
    if (!a) return GLA_B200_ERR_NULL;
    if ((a->K != 32 && a->K != gla::kD) || a->V != gla::kD || a->B < 0 || a->T < 0 || a->H < 0) return GLA_B200_ERR_SHAPE;
    if (a->direction < 0 || a->direction > 3) return GLA_B200_ERR_DIRECTION;
    int gh = a->grid_h, gw = a->grid_w;
    if (gh == 0 && gw == 0) { gh = 1; gw = a->T; }
    if (gh < 0 || gw < 0 || static_cast<int64_t>(gh) * gw != a->T) return GLA_B200_ERR_SHAPE;
    if (a->direction >= 2 && (a->grid_h <= 0 || a->grid_w <= 0)) return GLA_B200_ERR_SHAPE;
    if (a->scale != a->scale || a->gk_normalizer < 0.f) return GLA_B200_ERR_ARG;
    const bool gated = a->out_gate != nullptr || a->rms_weight != nullptr;
    if (gated && (!a->out_gate || !a->rms_weight)) return GLA_B200_ERR_NULL;
    if (gated && (!aligned16(a->out_gate) || !aligned16(a->rms_weight))) return GLA_B200_ERR_ALIGN;
    if (gated && !(a->rms_eps >= 0.f)) return GLA_B200_ERR_ARG;
    if (static_cast<int64_t>(a->B) * a->T * a->H == 0) {
        // nothing to compute; an empty sequence leaves the state as it came in
        const size_t state_bytes = static_cast<size_t>(a->B) * a->H * a->K * gla::kD * sizeof(float);
        if (a->final_state && state_bytes) {
            if (!aligned16(a->final_state) || (a->initial_state && !aligned16(a->initial_state))) return GLA_B200_ERR_ALIGN;
            cudaStream_t st = static_cast<cudaStream_t>(stream_v);
            cudaError_t e0 = a->initial_state
                                 ? cudaMemcpyAsync(a->final_state, a->initial_state, state_bytes, cudaMemcpyDeviceToDevice, st)
                                 : cudaMemsetAsync(a->final_state, 0, state_bytes, st);
            if (e0 != cudaSuccess) { note_cuda("final state of an empty sequence", e0); return GLA_B200_ERR_CUDA; }
        }
        return GLA_B200_OK;
    }
    if (!a->q || !a->k || !a->v || !a->g || !a->o) return GLA_B200_ERR_NULL;
    if (!aligned16(a->q) || !aligned16(a->k) || !aligned16(a->v) || !aligned16(a->g) || !aligned16(a->o) ||
        (a->initial_state && !aligned16(a->initial_state)) || (a->final_state && !aligned16(a->final_state)))
        return GLA_B200_ERR_ALIGN;
    if (a->segments < 0) return GLA_B200_ERR_ARG;

    MapKey key;
    memset(&key, 0, sizeof(key));
    const void* ptrs[gla::kNumTensors] = {a->q, a->k, a->g, a->v, a->o, nullptr};
    const int64_t* strides[gla::kNumTensors] = {a->q_stride, a->k_stride, a->g_stride, a->v_stride, a->o_stride,
                                                a->gate_stride};
    int rc = GLA_B200_OK;
    for (int t = 0; t < gla::kNumTensors; ++t) {
        key.ptr[t] = ptrs[t];
        if (!ptrs[t]) continue;
        const bool key_side = t == gla::TQ || t == gla::TK || t == gla::TG;
        rc = resolve_strides(strides[t], a->T, a->H, key_side ? a->K : gla::kD, key.stride[t]);
        if (rc != GLA_B200_OK) return rc;
    }

    int dev = 0;
    cudaError_t ce = cudaGetDevice(&dev);
    if (ce != cudaSuccess) { note_cuda("cudaGetDevice", ce); return GLA_B200_ERR_CUDA; }
    if (dev < 0 || dev >= 64) return GLA_B200_ERR_DEVICE;
    DeviceInfo di;
    rc = device_info(dev, &di);
    if (rc != GLA_B200_OK) return rc;
    const bool col = a->direction >= 2;
    key.B = a->B; key.T = a->T; key.H = a->H; key.K = a->K;
    key.col = col ? 1 : 0;
    key.Hc = col ? gh : a->T;
    key.Wc = col ? gw : 1;
    key.dev = dev;

    // segmentation
    const int NT = num_chunks(a->T);
    const int nseq = a->B * a->H;
    const int slots = gla::kCtasPerSm * di.sms;
    int cps;
    int plan_start[gla::kMaxPlanSegments + 1] = {0}, plan_ns = 0;
    bool plan = false, relay = false;
    if (a->segments > 0) cps = a->segments;
    else {
        const size_t have = a->workspace ? a->workspace_bytes : 0;
        cps = auto_chunks_per_segment(NT, nseq, slots, have);
        const int ns_u = (NT + cps - 1) / cps;
        const long rounds = (static_cast<long>(nseq) * ns_u + slots - 1) / slots;
        // what the slowest item of the equal split costs, in the plan's units: every segment but the last pays the pre-pass
        const double pre = gated ? kPlanPrePassGated : kPlanPrePassPlain;
        const double uniform_cost = rounds * (cps * (1.0 + (ns_u > 1 ? pre : 0.0)) + (ns_u > 1 ? 1.0 : 0.0));
        const double plan_cost = staggered_plan(NT, nseq, slots, have, pre, plan_start, &plan_ns);
        plan = plan_cost > 0.0 && plan_cost < uniform_cost;
        if (!plan && 2 * nseq > slots) {
            double relay_cost = 0.0;
            const int ns_r = relay_segments(NT, nseq, slots, have, &relay_cost);
            if (ns_r > 1 && relay_cost < 0.97 * uniform_cost) { relay = true; cps = (NT + ns_r - 1) / ns_r; }
        }
    }
    if (cps > NT) cps = NT;
    const int NS = plan ? plan_ns : (NT + cps - 1) / cps;
    const WsLayout L = ws_layout(static_cast<size_t>(nseq), static_cast<size_t>(NS));
    if (!a->workspace || (reinterpret_cast<uintptr_t>(a->workspace) & 255u) || a->workspace_bytes < L.total)
        return GLA_B200_ERR_WORKSPACE;

    gla::Maps maps;
    rc = get_maps(key, &maps);
    if (rc != GLA_B200_OK) return rc;

    uint8_t* ws = static_cast<uint8_t*>(a->workspace);
    gla::Params P;
    memset(&P, 0, sizeof(P));
    P.B = a->B; P.T = a->T; P.H = a->H; P.NT = NT; P.K = a->K;
    P.Hc = key.Hc; P.Wc = key.Wc;
    P.rev = a->direction & 1;
    P.NS = NS; P.cps = cps;
    P.plan = plan ? 1 : relay ? 2 : 0;
    for (int i = 0; i <= gla::kMaxPlanSegments; ++i) P.seg_start[i] = plan_start[i];
    P.num_items = nseq * NS;
    P.gated = gated ? 1 : 0;
    // q and k each carry sqrt(scale) / 4 (head-room for the gate factors in fp16); the 16 comes back in the epilogue
    if (a->scale > 0.f && a->scale < 3.0e38f) { P.q_exp = log2f(a->scale) - 4.f; P.q_mul = a->scale * 0.0625f; P.o_mul = 16.f; }
    else { P.q_exp = -4.f; P.q_mul = 0.0625f; P.o_mul = a->scale * 16.f; }
    P.inv_norm = a->gk_normalizer > 0.f ? 1.f / a->gk_normalizer : 0.f;
    P.rms_eps = a->rms_eps;
    P.rms_w = gated ? static_cast<const __half*>(a->rms_weight) : nullptr;
    P.gate = gated ? static_cast<const __half*>(a->out_gate) : nullptr;
    if (gated) {
        int64_t gs[3];
        rc = resolve_strides(a->gate_stride, a->T, a->H, gla::kD, gs);
        if (rc != GLA_B200_OK) return rc;
        P.gate_sb = gs[0]; P.gate_st = gs[1]; P.gate_sh = gs[2];
    }
    P.s0 = a->initial_state;
    P.sT = a->final_state;
    P.ctrl = reinterpret_cast<uint32_t*>(ws + L.ctrl);
    P.flags = reinterpret_cast<uint32_t*>(ws + L.flags);
    P.agg = reinterpret_cast<float*>(ws + L.agg);
    P.incl = reinterpret_cast<float*>(ws + L.incl);
    P.wait_limit_us = a->wait_limit ? a->wait_limit : 2000000u;
#ifdef GLA_TRACE
    P.trace = gla::g_trace_buffer;
#endif

    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    ce = cudaMemsetAsync(ws, 0, L.clear_bytes, stream);
    if (ce != cudaSuccess) { note_cuda("cudaMemsetAsync", ce); return GLA_B200_ERR_CUDA; }
    const int grid = P.num_items < slots ? P.num_items : slots;
    const int variant = (P.gated ? 4 : 0) | (P.inv_norm > 0.f ? 2 : 0) | (P.rev ? 1 : 0);
    void* kargs[2] = {const_cast<gla::Maps*>(&maps), &P};
    ce = cudaLaunchKernel(fwd_kernel(variant), dim3(grid), dim3(gla::kThreads), kargs, gla::kSmemBytes, stream);
    if (ce != cudaSuccess) { note_cuda("cudaLaunchKernel", ce); return GLA_B200_ERR_CUDA; }
    ce = cudaPeekAtLastError();
    if (ce != cudaSuccess) { note_cuda("kernel launch", ce); return GLA_B200_ERR_CUDA; }
    return GLA_B200_OK;
}

int gla_b200_stream_probe(const void* buf, int64_t rows, int32_t heads, int32_t ctas, int32_t tiles, int32_t chunks,
                          int32_t* status, void* stream_v) {
    if (!buf) return GLA_B200_ERR_NULL;
    if (heads <= 0 || ctas <= 0 || tiles < 1 || tiles > 4 || chunks <= 0 || rows <= 0) return GLA_B200_ERR_ARG;
    if (!aligned16(buf)) return GLA_B200_ERR_ALIGN;
    const int64_t slab_rows = rows / tiles;
    const int64_t regions = (ctas + heads - 1) / heads;
    if (regions * chunks * gla::kChunk > slab_rows || slab_rows * tiles > 0x7fffffffLL) return GLA_B200_ERR_ARG;
    int dev = 0;
    cudaError_t ce = cudaGetDevice(&dev);
    if (ce != cudaSuccess) { note_cuda("cudaGetDevice", ce); return GLA_B200_ERR_CUDA; }
    DeviceInfo di;
    int rc = device_info(dev, &di);
    if (rc != GLA_B200_OK) return rc;
    EncodeTiledFn enc = encode_tiled();
    if (!enc) return GLA_B200_ERR_DEVICE;
    CUtensorMap map;
    const cuuint64_t gdim[3] = {static_cast<cuuint64_t>(gla::kD), static_cast<cuuint64_t>(heads), static_cast<cuuint64_t>(rows)};
    const cuuint64_t gstr[2] = {static_cast<cuuint64_t>(gla::kD) * 2, static_cast<cuuint64_t>(heads) * gla::kD * 2};
    const cuuint32_t box[3] = {static_cast<cuuint32_t>(gla::kD), 1, static_cast<cuuint32_t>(gla::kChunk)}, estr[3] = {1, 1, 1};
    CUresult r = enc(&map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<void*>(buf), gdim, gstr, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { note_cu("cuTensorMapEncodeTiled", static_cast<int>(r)); return GLA_B200_ERR_CUDA; }
    const int smem = kProbeStages * gla::kStageBytes + 1024;
    static std::mutex mu;
    static bool attr[64] = {false};
    {
        std::lock_guard<std::mutex> lock(mu);
        if (dev >= 0 && dev < 64 && !attr[dev]) {
            ce = cudaFuncSetAttribute(stream_probe_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
            if (ce != cudaSuccess) { note_cuda("cudaFuncSetAttribute", ce); return GLA_B200_ERR_CUDA; }
            attr[dev] = true;
        }
    }
    stream_probe_kernel<<<ctas, kProbeThreads, smem, static_cast<cudaStream_t>(stream_v)>>>(
        map, heads, tiles, chunks, static_cast<int>(slab_rows), status);
    ce = cudaPeekAtLastError();
    if (ce != cudaSuccess) { note_cuda("stream probe launch", ce); return GLA_B200_ERR_CUDA; }
    return GLA_B200_OK;
}

int gla_b200_selftest_wait_timeout(void* workspace, size_t workspace_bytes, uint32_t limit_us, void* stream_v) {
    if (!workspace) {          // the built-in array of gla_b200_forward_static
        const int rc = static_scratch(&workspace);
        if (rc != GLA_B200_OK) return rc;
        workspace_bytes = GLA_B200_STATIC_SCRATCH_BYTES;
    }
    if ((reinterpret_cast<uintptr_t>(workspace) & 255u) || workspace_bytes < 512) return GLA_B200_ERR_WORKSPACE;
    if (limit_us == 0 || limit_us > 1000000u) return GLA_B200_ERR_ARG;      // a self-test never waits longer than 1 s
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    cudaError_t e = cudaMemsetAsync(workspace, 0, 512, stream);
    if (e != cudaSuccess) { note_cuda("cudaMemsetAsync", e); return GLA_B200_ERR_CUDA; }
    gla::Params P;
    memset(&P, 0, sizeof(P));
    P.ctrl = static_cast<uint32_t*>(workspace);
    P.flags = P.ctrl + 64;
    P.wait_limit_us = limit_us;
    gla::wait_timeout_selftest_kernel<<<1, 32, 0, stream>>>(P);
    e = cudaPeekAtLastError();
    if (e != cudaSuccess) { note_cuda("self-test launch", e); return GLA_B200_ERR_CUDA; }
    return GLA_B200_OK;
}

int gla_b200_check_status(const void* workspace, void* stream) {
    if (!workspace) {          // the built-in array of gla_b200_forward_static on the current device
        void* p = nullptr;
        const int rc = static_scratch(&p);
        if (rc != GLA_B200_OK) return rc;
        workspace = p;
    }
    uint32_t ctrl[2] = {0, 0};
    cudaError_t e = cudaMemcpyAsync(ctrl, workspace, sizeof(ctrl), cudaMemcpyDeviceToHost, static_cast<cudaStream_t>(stream));
    if (e == cudaSuccess) e = cudaStreamSynchronize(static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) { note_cuda("status read", e); return GLA_B200_ERR_CUDA; }
    return ctrl[1] == 0 ? GLA_B200_OK : GLA_B200_ERR_TIMEOUT;
}

// Segments per sequence for the gradient sweeps: enough CTAs to give every SM several (the sweeps hide latency by
// occupancy), segments of at least 256 tokens.  A pure function of the shape, so the workspace size can be asked ahead.
static int bwd_segments(int B, int T, int H, int* seg_len) {
    const int64_t ctas = 3LL * B * H;
    int nseg = static_cast<int>((600 + ctas - 1) / ctas);
    nseg = std::max(1, std::min(nseg, T / 256));
    int len = ((T + nseg - 1) / nseg + 31) / 32 * 32;
    nseg = (T + len - 1) / len;
    *seg_len = nseg > 1 ? len : std::max(T, 1);
    return nseg;
}

size_t gla_b200_backward_workspace_bytes(int32_t B, int32_t T, int32_t H, int32_t K, int32_t V) {
    if (B <= 0 || T <= 0 || H <= 0 || (K != 32 && K != 64) || V != 64) return 0;
    const size_t per = align_up(static_cast<size_t>(B) * T * H * K * sizeof(float), 256);
    int seg_len = 0;
    const size_t nseg = static_cast<size_t>(bwd_segments(B, T, H, &seg_len));
    const size_t seg = nseg > 1 ? align_up(2 * static_cast<size_t>(B) * H * nseg * K * (2 * 64 + 1) * sizeof(float), 256) : 0;
    return 2 * per + align_up(static_cast<size_t>(B) * H * K * sizeof(float), 256) + seg;
}

int gla_b200_backward(const gla_b200_bwd_args* a, void* stream_v) {
    if (!a) return GLA_B200_ERR_NULL;
    if (a->B < 0 || a->T < 0 || a->H <= 0 || (a->K != 32 && a->K != 64) || a->V != 64) return GLA_B200_ERR_SHAPE;
    if (static_cast<int64_t>(a->B) * a->H > 0x7fffffffLL) return GLA_B200_ERR_SHAPE;
    if (a->B == 0 || a->T == 0) return GLA_B200_OK;
    if (!a->q || !a->k || !a->v || !a->g || !a->d_o || !a->dq || !a->dk || !a->dv || !a->dg) return GLA_B200_ERR_NULL;
    const void* ptrs[] = {a->q, a->k, a->v, a->g, a->d_o, a->dq, a->dk, a->dv, a->dg, a->initial_state, a->d_final_state,
                          a->d_initial_state, a->workspace};
    for (const void* p : ptrs)
        if (p && !aligned16(p)) return GLA_B200_ERR_ALIGN;
    const size_t need = gla_b200_backward_workspace_bytes(a->B, a->T, a->H, a->K, a->V);
    if (!a->workspace || a->workspace_bytes < need) return GLA_B200_ERR_WORKSPACE;
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) { note_cuda("cudaGetDevice", e); return GLA_B200_ERR_CUDA; }
    DeviceInfo info;
    if (int rc = device_info(dev, &info)) return rc;

    gla::BwdParams P{};
    P.q = static_cast<const __half*>(a->q); P.k = static_cast<const __half*>(a->k); P.v = static_cast<const __half*>(a->v);
    P.g = static_cast<const __half*>(a->g); P.d_o = static_cast<const __half*>(a->d_o);
    P.dq = static_cast<__half*>(a->dq); P.dk = static_cast<__half*>(a->dk); P.dv = static_cast<__half*>(a->dv);
    P.dg = a->dg; P.h0 = a->initial_state; P.dht = a->d_final_state; P.dh0 = a->d_initial_state;
    const size_t per = align_up(static_cast<size_t>(a->B) * a->T * a->H * a->K * sizeof(float), 256);
    unsigned char* ws = static_cast<unsigned char*>(a->workspace);
    P.qdq = reinterpret_cast<float*>(ws); P.kdk = reinterpret_cast<float*>(ws + per);
    P.g_last = a->d_final_state ? reinterpret_cast<float*>(ws + 2 * per) : nullptr;
    P.B = a->B; P.T = a->T; P.H = a->H; P.scale = a->scale;
    P.nseg = bwd_segments(a->B, a->T, a->H, &P.seg_len);
    const size_t last = align_up(static_cast<size_t>(a->B) * a->H * a->K * sizeof(float), 256);
    P.seg_state = reinterpret_cast<float*>(ws + 2 * per + last);
    P.seg_start = P.seg_state + 2 * static_cast<size_t>(a->B) * a->H * P.nseg * a->K * 64;
    P.seg_decay = P.seg_start + 2 * static_cast<size_t>(a->B) * a->H * P.nseg * a->K * 64;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    const unsigned bh = static_cast<unsigned>(a->B * a->H);
    if (static_cast<int64_t>(bh) * P.nseg > 0x7fffffffLL) return GLA_B200_ERR_SHAPE;
#define GLA_BWD_LAUNCH(KK)                                                                                            \
    do {                                                                                                              \
        if (P.nseg > 1) {                                                                                             \
            gla::gla_bwd_state_kernel<KK><<<dim3(bh * (P.nseg - 1), 2), gla::kBwdThreads, 0, stream>>>(P);            \
            gla::gla_bwd_combine_kernel<KK><<<dim3(bh, 2, KK / 4), 256, 0, stream>>>(P);                                   \
        }                                                                                                             \
        gla::gla_bwd_sweep_kernel<KK><<<dim3(bh * P.nseg, 3), gla::kBwdThreads, 0, stream>>>(P);                      \
        if (bh >= 256) gla::gla_bwd_dg_kernel<KK, KK><<<dim3(bh, 1), 1024, 0, stream>>>(P);                           \
        else gla::gla_bwd_dg_kernel<KK, 16><<<dim3(bh, KK / 16), 1024, 0, stream>>>(P);                               \
    } while (0)
    if (a->K == 64) GLA_BWD_LAUNCH(64);
    else GLA_BWD_LAUNCH(32);
#undef GLA_BWD_LAUNCH
    e = cudaPeekAtLastError();
    if (e != cudaSuccess) { note_cuda("backward launch", e); return GLA_B200_ERR_CUDA; }
    return GLA_B200_OK;
}

int gla_b200_rmsnorm_gated(const void* x, const void* g, const void* w, void* y, int64_t rows, int32_t D, float eps,
                           void* stream) {
    if (D != 64 || rows < 0) return GLA_B200_ERR_SHAPE;
    if (rows == 0) return GLA_B200_OK;
    if (!x || !g || !w || !y) return GLA_B200_ERR_NULL;
    if (!aligned16(x) || !aligned16(g) || !aligned16(w) || !aligned16(y)) return GLA_B200_ERR_ALIGN;
    const int64_t threads = rows * 8;
    const int64_t blocks = (threads + 255) / 256;
    if (blocks > 0x7fffffffLL) return GLA_B200_ERR_SHAPE;
    rmsnorm_gated_kernel<<<static_cast<unsigned>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __half*>(x), static_cast<const __half*>(g), static_cast<const __half*>(w),
        static_cast<__half*>(y), rows, eps);
    cudaError_t e = cudaPeekAtLastError();
    if (e != cudaSuccess) { note_cuda("rmsnorm launch", e); return GLA_B200_ERR_CUDA; }
    return GLA_B200_OK;
}

int gla_b200_swiglu_dwconv(const void* gate, const void* y, const void* weight, const void* bias, void* out,
                           int32_t B, int32_t grid_h, int32_t grid_w, int32_t C, void* stream) {
    if (B < 0 || grid_h < 0 || grid_w < 0 || C <= 0 || (C & 7)) return GLA_B200_ERR_SHAPE;
    if (static_cast<int64_t>(B) * grid_h * grid_w == 0) return GLA_B200_OK;
    if (!gate || !y || !weight || !out) return GLA_B200_ERR_NULL;
    if (!aligned16(gate) || !aligned16(y) || !aligned16(weight) || !aligned16(out) || (bias && !aligned16(bias)))
        return GLA_B200_ERR_ALIGN;
    if (out == gate || out == y) return GLA_B200_ERR_ARG;      // neighbours are read after their own output is written
    {
        const int64_t tiles = static_cast<int64_t>((grid_h + gla::kDwTileR - 1) / gla::kDwTileR) *
                              ((grid_w + gla::kDwTileC - 1) / gla::kDwTileC);
        const int64_t blocks = static_cast<int64_t>(B) * tiles * (((C >> 3) + gla::kDwSlab - 1) / gla::kDwSlab);
        if (blocks > 0x7fffffffLL) return GLA_B200_ERR_SHAPE;
        gla::swiglu_dwconv_kernel<<<static_cast<unsigned>(blocks), gla::kDwTileThreads, gla::kDwTileSmem,
                                          static_cast<cudaStream_t>(stream)>>>(
            static_cast<const __half*>(gate), static_cast<const __half*>(y), static_cast<const __half*>(weight),
            static_cast<const __half*>(bias), static_cast<__half*>(out), B, grid_h, grid_w, C);
    }
    cudaError_t e = cudaPeekAtLastError();
    if (e != cudaSuccess) { note_cuda("swiglu_dwconv launch", e); return GLA_B200_ERR_CUDA; }
    return GLA_B200_OK;
}

int gla_b200_layernorm(const void* x, const void* weight, const void* bias, void* y, int64_t rows, int32_t D, float eps,
                       void* stream) {
    if (rows < 0 || D <= 0 || (D & 7) || D > 256 * gla::kLnMaxVec) return GLA_B200_ERR_SHAPE;
    if (rows == 0) return GLA_B200_OK;
    if (!x || !weight || !y) return GLA_B200_ERR_NULL;
    if (!aligned16(x) || !aligned16(weight) || !aligned16(y) || (bias && !aligned16(bias))) return GLA_B200_ERR_ALIGN;
    const int64_t blocks = (rows + 7) / 8;               // eight warps, one row each
    if (blocks > 0x7fffffffLL) return GLA_B200_ERR_SHAPE;
    const int per_lane = ((D >> 3) + 31) / 32;            // 16-byte vectors per lane
#define GLA_LN_LAUNCH(V)                                                                                              \
    gla::layernorm_rows_kernel<V><<<static_cast<unsigned>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(      \
        static_cast<const __half*>(x), static_cast<const __half*>(weight), static_cast<const __half*>(bias),          \
        static_cast<__half*>(y), rows, D, eps)
    if (per_lane <= 1) GLA_LN_LAUNCH(1);
    else if (per_lane <= 2) GLA_LN_LAUNCH(2);
    else if (per_lane <= 3) GLA_LN_LAUNCH(3);
    else if (per_lane <= 4) GLA_LN_LAUNCH(4);
    else GLA_LN_LAUNCH(gla::kLnMaxVec);
#undef GLA_LN_LAUNCH
    cudaError_t e = cudaPeekAtLastError();
    if (e != cudaSuccess) { note_cuda("layernorm launch", e); return GLA_B200_ERR_CUDA; }
    return GLA_B200_OK;
}

int32_t gla_b200_trt_enqueue(const void* const* inputs, int32_t n_inputs, void* const* outputs, const int64_t* q_dims,
                             float scale, float gk_normalizer, float rms_eps, void* workspace, size_t workspace_bytes,
                             void* stream) {
    if (!inputs || !outputs || !q_dims || !workspace || (n_inputs != 4 && n_inputs != 6)) return -1;
    gla_b200_args a;
    memset(&a, 0, sizeof(a));
    a.q = inputs[0]; a.k = inputs[1]; a.v = inputs[2]; a.g = inputs[3];
    a.o = outputs[0];
    const bool fused = n_inputs == 6 && rms_eps > 0.f;
    if (fused) { a.out_gate = inputs[4]; a.rms_weight = inputs[5]; a.rms_eps = rms_eps; }
    a.B = static_cast<int32_t>(q_dims[0]); a.T = static_cast<int32_t>(q_dims[1]);
    a.H = static_cast<int32_t>(q_dims[2]); a.K = static_cast<int32_t>(q_dims[3]);
    a.V = GLA_B200_HEAD_V;
    a.scale = scale;
    a.gk_normalizer = gk_normalizer;
    // TensorRT hands out workspaces with its own alignment; round up to ours like the reference plugin does
    uintptr_t p = (reinterpret_cast<uintptr_t>(workspace) + 255u) & ~static_cast<uintptr_t>(255u);
    const size_t lost = p - reinterpret_cast<uintptr_t>(workspace);
    if (workspace_bytes < lost) return -1;
    a.workspace = reinterpret_cast<void*>(p);
    a.workspace_bytes = workspace_bytes - lost;
    return gla_b200_forward(&a, stream) == GLA_B200_OK ? 0 : -1;
}

}  // extern "C"

extern "C" int gla_b200_forward_static(const gla_b200_args* a, void* stream) {
    if (!a) return GLA_B200_ERR_NULL;
    void* ptr = nullptr;
    const int rc0 = static_scratch(&ptr);
    if (rc0 != GLA_B200_OK) return rc0;
    gla_b200_args b = *a;
    b.workspace = ptr;
    b.workspace_bytes = GLA_B200_STATIC_SCRATCH_BYTES;
    // The automatic policy only considers segmentations whose scratch fits the array; only an explicit
    // `segments` can ask for more than it holds.
    const int rc = gla_b200_forward(&b, stream);
    return rc == GLA_B200_ERR_WORKSPACE ? GLA_B200_ERR_STATIC_SCRATCH : rc;
}
