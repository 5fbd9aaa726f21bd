/*
 * gla_b200 -- C ABI of the B200 (sm_100a) chunkwise gated-linear-attention forward operator.
 *
 * Plain pointers and sizes only: this is the boundary a host in any language binds to
 * (ctypes, pybind, a TensorRT plugin's enqueue).  Each entry point names the interface of
 * the GTR reference it stands in for (paths relative to the GTR project root).
 *
 * Tensor contract (reference: engine/gtr/backbone/csrc/gla_torch_ext.cu:15-22,49-66):
 *   q, k, g : fp16 [B, T, H, K]      v, o, out_gate : fp16 [B, T, H, V]      K = 32 or 64, V = 64
 *   (K = 32, V = 64 is the reference extension's only shape, gla_chunk.cuh:14-16, and what the released GTR
 *   configs use; K = 64 is what its FLA path serves at expand_k = 1.)
 *   g is the log-space forget gate (<= 0), or raw logits when gk_normalizer > 0, in which
 *   case the kernel applies logsigmoid(g) / gk_normalizer (gla_chunk.cuh:775,788-790).
 *   States are fp32 [B, H, K, V].  All pointers are device pointers, 16-byte aligned.
 *   Unlike the reference, tensors need not be contiguous: each has element strides for
 *   (batch, token, head); the innermost dimension must be dense.  A stride triple of
 *   {0,0,0} means contiguous.  Strides must be multiples of 8 elements (16 bytes).
 *
 * Recurrence computed, per batch b and head h, along the scan order p = 0..T-1:
 *   S_p = exp(g_p)[:,None] * S_{p-1} + k_p v_p^T ,   o_p = scale * q_p^T S_p
 * `direction` selects which token each step p reads on the grid_h x grid_w patch grid
 * (reference: engine/gtr/backbone/vit_adapter_spatial_swiglu.py:88-94, the physical token
 * permutation applied between backbone blocks; here it is folded into the tile coordinates):
 *   0 row-major, 1 row-major reversed, 2 column-major, 3 column-major reversed.
 *   Outputs are written at the token's own (unpermuted) position.
 */
#ifndef GLA_B200_H_
#define GLA_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define GLA_B200_VERSION 1
#define GLA_B200_CHUNK 64          /* tokens per chunk; reference kBT, gla_chunk.cuh:16 */
#define GLA_B200_HEAD_K 64         /* widest key head; K = 32 (reference kK, gla_chunk.cuh:14) is served too */
#define GLA_B200_HEAD_V 64         /* reference kV, gla_chunk.cuh:15 */

enum gla_b200_direction {
    GLA_B200_ROW = 0, GLA_B200_ROW_REV = 1, GLA_B200_COL = 2, GLA_B200_COL_REV = 3
};

enum gla_b200_error {
    GLA_B200_OK = 0,
    GLA_B200_ERR_NULL = -1,          /* a required pointer is NULL */
    GLA_B200_ERR_SHAPE = -2,         /* unsupported B/T/H/K/V or grid_h*grid_w != T */
    GLA_B200_ERR_ALIGN = -3,         /* pointer or stride not 16-byte aligned */
    GLA_B200_ERR_DIRECTION = -4,     /* direction outside 0..3 */
    GLA_B200_ERR_WORKSPACE = -5,     /* workspace missing or smaller than gla_b200_workspace_bytes */
    GLA_B200_ERR_DEVICE = -6,        /* not an sm_100 device, or driver entry point unavailable */
    GLA_B200_ERR_CUDA = -7,          /* a CUDA runtime/driver call failed (see gla_b200_last_cuda_error) */
    GLA_B200_ERR_TIMEOUT = -8,       /* device status word: a bounded wait inside the kernel expired */
    GLA_B200_ERR_ARG = -9,           /* any other invalid argument */
    GLA_B200_ERR_STATIC_SCRATCH = -10 /* gla_b200_forward_static: problem exceeds the built-in scratch array */
};

typedef struct gla_b200_args {
    const void* q;
    const void* k;
    const void* v;
    const void* g;
    void* o;
    /* optional: fused RMSNorm * weight * silu(out_gate) epilogue (reference chunk_gla_run_gated,
     * gla_torch_ext.cu:92-154); both NULL for the plain operator */
    const void* out_gate;
    const void* rms_weight;          /* fp16 [V] */
    /* optional fp32 [B,H,K,V] states (FLA call signature, vit_adapter.py:566-568) */
    const float* initial_state;
    float* final_state;
    /* caller-owned scratch, >= gla_b200_workspace_bytes(B,T,H,K,V), 256-byte aligned */
    void* workspace;
    size_t workspace_bytes;
    int64_t q_stride[3], k_stride[3], v_stride[3], g_stride[3], o_stride[3], gate_stride[3];
    int32_t B, T, H, K, V;
    int32_t grid_h, grid_w;          /* patch grid; needed for directions 2,3; 0,0 means 1 x T */
    int32_t direction;
    int32_t segments;                /* chunks of one sequence handled per work item; 0 = automatic */
    float scale;                     /* applied to the output, reference default K^-0.5 */
    float gk_normalizer;             /* 0: g is a log gate; >0: g holds logits */
    float rms_eps;
    uint32_t wait_limit;             /* microseconds before a device-side wait gives up; 0 = 2 s */
} gla_b200_args;

/* Replaces chunk_gla_run / chunk_gla_run_gated (gla_torch_ext.cu:40-154) and
 * gla_chunk::launch_chunk_gla (gla_chunk.cuh:1446-1540).  Enqueues on `stream`
 * (a cudaStream_t), never synchronises, never allocates; capturable in a CUDA graph once
 * the calling thread has run the same shape once.  Returns 0 or a gla_b200_error. */
int gla_b200_forward(const gla_b200_args* args, void* stream);

/* Same operator, but with nothing allocated and no workspace from the caller (`workspace` and
 * `workspace_bytes` of `args` are ignored): the scratch is a fixed array of
 * GLA_B200_STATIC_SCRATCH_BYTES inside the library, one per GPU, held until the process exits.
 * It is meant for callers that cannot reach the device allocator at call time -- a server whose
 * memory pool owns the whole GPU, a plugin that is handed no workspace, a loop with a frozen memory
 * budget.  No counterpart in the reference (its callers always bring a workspace tensor).
 * The first call on a device looks up the array's device address; issue it before any stream
 * capture.  The array is shared by all calls on that GPU and keeps the last call's contents (the
 * words that must be zero are cleared at the start of each call), so calls that overlap on one GPU
 * race: run them one after another.  The automatic segmentation (`segments` = 0) only considers splits whose
 * scratch fits the array and settles for a coarser one otherwise (one work item per sequence needs no
 * scratch beyond the control words), so it never fails for size; an explicit `segments` that needs more
 * than the array returns GLA_B200_ERR_STATIC_SCRATCH.  A time-out inside such a call is read with
 * gla_b200_check_status(NULL, stream). */
#define GLA_B200_STATIC_SCRATCH_BYTES (24u << 20)
int gla_b200_forward_static(const gla_b200_args* args, void* stream);

/* Replaces workspace_floats (gla_torch_ext.cu:24-33); bytes, not floats.  0 on bad shape. */
size_t gla_b200_workspace_bytes(int32_t B, int32_t T, int32_t H, int32_t K, int32_t V);

/* Reads the device status word of a workspace after synchronising `stream`:
 * 0, or GLA_B200_ERR_TIMEOUT when a bounded wait expired during the last forward.
 * `workspace` == NULL reads the status of the current device's built-in array, i.e. of the last
 * gla_b200_forward_static call there.
 * The reference has no counterpart (its waits are unbounded, gla_chunk.cuh:1229-1233). */
int gla_b200_check_status(const void* workspace, void* stream);

/* Exercises the kernel's bounded waits without any real work: one warp waits on a barrier and on a
 * flag that nothing ever completes, with a limit of `limit_us` microseconds (<= 1 s).  Afterwards
 * gla_b200_check_status(workspace) must report GLA_B200_ERR_TIMEOUT and the context stays usable.
 * `workspace` == NULL runs the test on the built-in array of gla_b200_forward_static.
 * No counterpart in the reference, whose device-side waits are unbounded. */
int gla_b200_selftest_wait_timeout(void* workspace, size_t workspace_bytes, uint32_t limit_us, void* stream);

/* Diagnostic: what the kernel's way of loading -- a ring of five stages of 64-row x 128-byte tiles per CTA, filled by
 * TMA from a [rows, heads, 64] fp16 tensor with one head per CTA -- can stream on this GPU when nothing is computed.
 * `ctas` CTAs (one per SM) each read `chunks` chunks of `tiles` tiles (3 = the pre-pass's k, g, v; 4 = the output
 * pass's q, k, g, v) from their own rows of `buf`; the stage is handed back as soon as it has landed.  The caller times
 * the call with events: bytes = ctas * chunks * tiles * 8192.  `status` (device, one int, may be NULL) is set to a
 * non-zero value if a bounded wait gave up.  `buf` needs rows >= tiles * (ctas / heads + 1) * chunks * 64.
 * bench.py reports the figure beside the roofline as the ceiling of the loading scheme itself; the reference has no
 * counterpart. */
int gla_b200_stream_probe(const void* buf, int64_t rows, int32_t heads, int32_t ctas, int32_t tiles, int32_t chunks,
                          int32_t* status, void* stream);

/* Gradient of the plain operator (row-major scan, log-space gates), for training.  The reference has no CUDA gradient
 * of its own: its training path calls the third-party FLA operator and relies on that operator's autograd
 * (engine/gtr/backbone/vit_adapter.py:441,560-568; flash-linear-attention 0.5.0, requirements.txt:9).  This entry point
 * is what an autograd wrapper around gla_b200_forward calls in its backward.
 *   q, k, g : fp16 [B,T,H,K]   v, d_o : fp16 [B,T,H,V]   contiguous   ->   dq, dk : fp16 [B,T,H,K]   dv : fp16 [B,T,H,V]
 *   dg : fp32 [B,T,H,K] (the caller casts)   states and their gradients: fp32 [B,H,K,V], each optional (NULL).
 * With S_t = exp(g_t) S_{t-1} + k_t v_t^T, o_t = scale q_t^T S_t:
 *   dS_t = exp(g_{t+1}) dS_{t+1} + scale q_t do_t^T,  dq_t = scale S_t do_t,  dk_t = dS_t v_t,  dv_t = dS_t^T k_t,
 *   dg_t = sum_{s>=t} (q_s dq_s - k_s dk_s) (+ sum_v d_final_state * final_state at the last token),
 *   d_initial_state = exp(g_1) dS_1.
 * Never synchronises or allocates; the workspace needs no clearing. */
typedef struct gla_b200_bwd_args {
    const void* q;
    const void* k;
    const void* v;
    const void* g;
    const void* d_o;
    void* dq;
    void* dk;
    void* dv;
    float* dg;
    const float* initial_state;      /* the forward call's initial state, or NULL */
    const float* d_final_state;      /* gradient flowing into the forward call's final state, or NULL */
    float* d_initial_state;          /* out, or NULL */
    void* workspace;                 /* >= gla_b200_backward_workspace_bytes(B,T,H,K,V), 256-byte aligned */
    size_t workspace_bytes;
    int32_t B, T, H, K, V;
    float scale;
} gla_b200_bwd_args;

size_t gla_b200_backward_workspace_bytes(int32_t B, int32_t T, int32_t H, int32_t K, int32_t V);
int gla_b200_backward(const gla_b200_bwd_args* args, void* stream);

/* Replaces rmsnorm_gated (gla_torch_ext.cu:156-196, kernel gla_norm_gate.cuh:13-75):
 * y = x * rsqrt(mean(x^2) + eps) * w * silu(g) over rows of D = 64 fp16 values; y may alias x. */
int gla_b200_rmsnorm_gated(const void* x, const void* g, const void* w, void* y,
                           int64_t rows, int32_t D, float eps, void* stream);

/* Middle step of the backbone's Spatial SwiGLU MLP in its deploy form
 * (engine/gtr/backbone/vit_adapter_spatial_swiglu.py:50-60: view as grid -> 3x3 depthwise conv -> view back ->
 * silu(gate) * y), in one pass:  out = silu(gate) * (bias + dwconv3x3(y))  on tokens laid out [B, grid_h*grid_w, C],
 * zero padding at the grid border.  gate, y, out: fp16 [B, grid_h*grid_w, C] contiguous, out distinct from both;
 * weight: fp16 [3][3][C] (tap-major: the reference's [C,1,3,3] weight permuted, already oriented for the
 * canonical grid); bias: fp16 [C] or NULL.  C a multiple of 8. */
int gla_b200_swiglu_dwconv(const void* gate, const void* y, const void* weight, const void* bias, void* out,
                           int32_t B, int32_t grid_h, int32_t grid_w, int32_t C, void* stream);

/* LayerNorm over rows of D fp16 values with fp32 statistics: y = (x - mean) * rsqrt(var + eps) * weight + bias.
 * The norms in front of the backbone block's attention and MLP (engine/gtr/backbone/vit_adapter.py:608-642, nn.LayerNorm
 * with eps 1e-6) in one read and one write of the activations.  D a multiple of 8, at most 2048; bias may be NULL;
 * y may alias x. */
int gla_b200_layernorm(const void* x, const void* weight, const void* bias, void* y, int64_t rows, int32_t D, float eps,
                       void* stream);

/* Shape of GLAPlugin::enqueue (tensorrt_plugin/trt_plugin/gla_plugin.cu:124-163): `inputs` holds
 * q,k,v,gk[,g,rms_w] device pointers, `outputs[0]` the result, dims are those of q [B,T,H,K];
 * the fused epilogue is used iff n_inputs == 6 and rms_eps > 0 (gla_plugin.cu:150).
 * Returns 0 or -1 like the plugin. */
int32_t gla_b200_trt_enqueue(const void* const* inputs, int32_t n_inputs, void* const* outputs,
                             const int64_t* q_dims, float scale, float gk_normalizer, float rms_eps,
                             void* workspace, size_t workspace_bytes, void* stream);

const char* gla_b200_strerror(int code);
const char* gla_b200_last_cuda_error(void);
int gla_b200_version(void);

#ifdef __cplusplus
}
#endif
#endif /* GLA_B200_H_ */
