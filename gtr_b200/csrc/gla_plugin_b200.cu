// TensorRT plugin "GatedLinearAttention" version "1" on top of libgla_b200.so.
//
// Same contract as the reference plugin (tensorrt_plugin/trt_plugin/gla_plugin.cu:19-20,54-209): plugin name
// `GatedLinearAttention`, version `1`, empty namespace; creator fields `scale`, `gk_normalizer`, `rms_eps`
// (one FLOAT32 each; the ONNX node carries them as scale_f / gk_normalizer_f / rms_eps_f,
// tensorrt_plugin/gtr_onnx_patches.py:72-90); inputs q, k, v, gk [, g, rms_w], all LINEAR + HALF; one output shaped
// and typed like v; the fused RMSNorm * w * silu(g) epilogue is taken iff six inputs are bound and rms_eps > 0
// (gla_plugin.cu:150).  What differs: `enqueue` hands the pointers to gla_b200_trt_enqueue (one persistent sm_100a
// kernel) and the workspace is what gla_b200_workspace_bytes asks for, a few MB instead of the reference layout's
// fp32 copies of G, S and h.  K = 32 and K = 64 key heads are accepted.
//
// The file compiles only where TensorRT's headers are found; a build without them yields an empty object, and
// nothing else in the library depends on it.
#if defined(__has_include)
#if __has_include(<NvInfer.h>)
#define GLA_B200_HAVE_TENSORRT 1
#endif
#endif

#ifdef GLA_B200_HAVE_TENSORRT
#include <NvInfer.h>
#include <cuda_runtime_api.h>

#include <cstdint>
#include <cstring>
#include <new>
#include <vector>

#include "gla_b200.h"

namespace gla_b200_trt {

using namespace nvinfer1;

constexpr char const* kName = "GatedLinearAttention";
constexpr char const* kVersion = "1";
constexpr size_t kAlignSlack = 256;      // TensorRT's workspace alignment is its own; the enqueue shim rounds up

struct Settings {
    float scale = 1.0f;
    float gk_normalizer = 0.0f;
    float rms_eps = 0.0f;
};

// One table drives the creator's advertised fields, their parsing and the serialised form.
struct Attr {
    char const* name;
    float Settings::*member;
};
constexpr Attr kAttrs[] = {{"scale", &Settings::scale}, {"gk_normalizer", &Settings::gk_normalizer},
                           {"rms_eps", &Settings::rms_eps}};
constexpr int32_t kNumAttrs = static_cast<int32_t>(sizeof(kAttrs) / sizeof(kAttrs[0]));

inline bool shape_bthd(Dims const& d) { return d.nbDims == 4; }

class Plugin final : public IPluginV3, public IPluginV3OneCore, public IPluginV3OneBuild, public IPluginV3OneRuntime {
public:
    explicit Plugin(Settings const& s) : settings_(s) { rebuild_fields(); }
    Plugin(Plugin const& other) : settings_(other.settings_) { rebuild_fields(); }
    Plugin& operator=(Plugin const&) = delete;

    // IPluginV3
    IPluginCapability* getCapabilityInterface(PluginCapabilityType type) noexcept override {
        switch (type) {
            case PluginCapabilityType::kBUILD: return static_cast<IPluginV3OneBuild*>(this);
            case PluginCapabilityType::kRUNTIME: return static_cast<IPluginV3OneRuntime*>(this);
            default: return static_cast<IPluginV3OneCore*>(this);
        }
    }
    IPluginV3* clone() noexcept override { return new (std::nothrow) Plugin(*this); }

    // IPluginV3OneCore
    char const* getPluginName() const noexcept override { return kName; }
    char const* getPluginVersion() const noexcept override { return kVersion; }
    char const* getPluginNamespace() const noexcept override { return ""; }

    // IPluginV3OneBuild
    int32_t getNbOutputs() const noexcept override { return 1; }
    int32_t configurePlugin(DynamicPluginTensorDesc const*, int32_t nb_inputs, DynamicPluginTensorDesc const*,
                            int32_t nb_outputs) noexcept override {
        return ((nb_inputs == 4 || nb_inputs == 6) && nb_outputs == 1) ? 0 : -1;
    }
    bool supportsFormatCombination(int32_t pos, DynamicPluginTensorDesc const* in_out, int32_t nb_inputs,
                                   int32_t nb_outputs) noexcept override {
        if (pos < 0 || pos >= nb_inputs + nb_outputs) return false;
        PluginTensorDesc const& d = in_out[pos].desc;
        return d.type == DataType::kHALF && d.format == TensorFormat::kLINEAR;
    }
    int32_t getOutputDataTypes(DataType* out_types, int32_t nb_outputs, DataType const* in_types,
                               int32_t nb_inputs) const noexcept override {
        if (nb_outputs != 1 || nb_inputs < 3) return -1;
        out_types[0] = in_types[2];
        return 0;
    }
    int32_t getOutputShapes(DimsExprs const* inputs, int32_t nb_inputs, DimsExprs const*, int32_t, DimsExprs* outputs,
                            int32_t nb_outputs, IExprBuilder&) noexcept override {
        if (nb_inputs < 3 || nb_outputs != 1) return -1;
        outputs[0] = inputs[2];                       // [B, T, H, V], the shape of v
        return 0;
    }
    size_t getWorkspaceSize(DynamicPluginTensorDesc const* inputs, int32_t nb_inputs, DynamicPluginTensorDesc const*,
                            int32_t) const noexcept override {
        if (nb_inputs < 3 || !shape_bthd(inputs[0].max) || !shape_bthd(inputs[2].max)) return 0;
        Dims const& q = inputs[0].max;                // the largest shape of the profile; static in GTR's engines
        const size_t need = gla_b200_workspace_bytes(static_cast<int32_t>(q.d[0]), static_cast<int32_t>(q.d[1]),
                                                     static_cast<int32_t>(q.d[2]), static_cast<int32_t>(q.d[3]),
                                                     static_cast<int32_t>(inputs[2].max.d[3]));
        return need ? need + kAlignSlack : 0;
    }

    // IPluginV3OneRuntime
    int32_t onShapeChange(PluginTensorDesc const* in, int32_t nb_inputs, PluginTensorDesc const*, int32_t) noexcept override {
        bound_inputs_ = nb_inputs;
        if (nb_inputs >= 1 && shape_bthd(in[0].dims)) {
            // remember the workspace size the engine was asked for: enqueue is not told
            workspace_bytes_ = gla_b200_workspace_bytes(
                static_cast<int32_t>(in[0].dims.d[0]), static_cast<int32_t>(in[0].dims.d[1]),
                static_cast<int32_t>(in[0].dims.d[2]), static_cast<int32_t>(in[0].dims.d[3]), GLA_B200_HEAD_V) + kAlignSlack;
        }
        return 0;
    }
    IPluginV3* attachToContext(IPluginResourceContext*) noexcept override { return clone(); }
    PluginFieldCollection const* getFieldsToSerialize() noexcept override { return &serialised_; }

    int32_t enqueue(PluginTensorDesc const* in_desc, PluginTensorDesc const*, void const* const* inputs,
                    void* const* outputs, void* workspace, cudaStream_t stream) noexcept override {
        if (!in_desc || !inputs || !outputs || !workspace) return -1;
        Dims const& q = in_desc[0].dims;
        Dims const& v = in_desc[2].dims;
        if (!shape_bthd(q) || !shape_bthd(v) || in_desc[0].type != DataType::kHALF) return -1;
        if (v.d[3] != GLA_B200_HEAD_V) return -1;
        const int64_t dims[4] = {q.d[0], q.d[1], q.d[2], q.d[3]};
        const int32_t n = (bound_inputs_ == 6 && settings_.rms_eps > 0.0f) ? 6 : 4;
        size_t ws = workspace_bytes_;
        if (ws == 0)
            ws = gla_b200_workspace_bytes(static_cast<int32_t>(q.d[0]), static_cast<int32_t>(q.d[1]),
                                          static_cast<int32_t>(q.d[2]), static_cast<int32_t>(q.d[3]), GLA_B200_HEAD_V) +
                 kAlignSlack;
        return gla_b200_trt_enqueue(inputs, n, outputs, dims, settings_.scale, settings_.gk_normalizer,
                                    settings_.rms_eps, workspace, ws, stream);
    }

private:
    void rebuild_fields() {
        fields_.clear();
        for (Attr const& a : kAttrs) fields_.push_back(PluginField{a.name, &(settings_.*a.member), PluginFieldType::kFLOAT32, 1});
        serialised_.nbFields = kNumAttrs;
        serialised_.fields = fields_.data();
    }

    Settings settings_;
    int32_t bound_inputs_ = 4;
    size_t workspace_bytes_ = 0;
    std::vector<PluginField> fields_;
    PluginFieldCollection serialised_{};
};

class Creator final : public IPluginCreatorV3One {
public:
    Creator() {
        for (Attr const& a : kAttrs) names_.push_back(PluginField{a.name, nullptr, PluginFieldType::kFLOAT32, 1});
        advertised_.nbFields = kNumAttrs;
        advertised_.fields = names_.data();
    }
    char const* getPluginName() const noexcept override { return kName; }
    char const* getPluginVersion() const noexcept override { return kVersion; }
    char const* getPluginNamespace() const noexcept override { return ""; }
    PluginFieldCollection const* getFieldNames() noexcept override { return &advertised_; }

    IPluginV3* createPlugin(char const*, PluginFieldCollection const* fc, TensorRTPhase) noexcept override {
        Settings s;
        const int32_t n = (fc && fc->fields) ? fc->nbFields : 0;
        for (int32_t i = 0; i < n; ++i) {
            PluginField const& f = fc->fields[i];
            if (!f.name || !f.data) continue;
            float value;
            if (f.type == PluginFieldType::kFLOAT32) value = *static_cast<float const*>(f.data);
            else if (f.type == PluginFieldType::kFLOAT64) value = static_cast<float>(*static_cast<double const*>(f.data));
            else continue;
            for (Attr const& a : kAttrs)
                if (std::strcmp(f.name, a.name) == 0) s.*a.member = value;
        }
        return new (std::nothrow) Plugin(s);
    }

private:
    std::vector<PluginField> names_;
    PluginFieldCollection advertised_{};
};

REGISTER_TENSORRT_PLUGIN(Creator);

}  // namespace gla_b200_trt

// Lets a host (or a test) reach the creator without going through TensorRT's registry.
extern "C" nvinfer1::IPluginCreatorV3One* gla_b200_trt_plugin_creator() {
    static gla_b200_trt::Creator creator;
    return &creator;
}
#endif  // GLA_B200_HAVE_TENSORRT
