// Exercises gla_plugin_b200.cu against the stand-in NvInfer.h (no TensorRT, no GPU): creator -> plugin with fields
// -> name / version / field round trip / format checks / workspace size / clone.  Prints one line per check and
// returns the number of failures.
#include <cstdio>
#include <cstring>

#include "NvInfer.h"
#include "gla_b200.h"

extern "C" nvinfer1::IPluginCreatorV3One* gla_b200_trt_plugin_creator();

using namespace nvinfer1;

static int failures = 0;
#define CHECK(cond) do { const bool ok_ = (cond); std::printf("%s %s\n", ok_ ? "ok  " : "FAIL", #cond); if (!ok_) ++failures; } while (0)

static DynamicPluginTensorDesc desc(int64_t b, int64_t t, int64_t h, int64_t d, DataType type = DataType::kHALF,
                                    TensorFormat fmt = TensorFormat::kLINEAR) {
    DynamicPluginTensorDesc x{};
    x.desc.dims.nbDims = 4;
    x.desc.dims.d[0] = b; x.desc.dims.d[1] = t; x.desc.dims.d[2] = h; x.desc.dims.d[3] = d;
    x.desc.type = type;
    x.desc.format = fmt;
    x.min = x.opt = x.max = x.desc.dims;
    return x;
}

int main() {
    IPluginCreatorV3One* creator = gla_b200_trt_plugin_creator();
    CHECK(std::strcmp(creator->getPluginName(), "GatedLinearAttention") == 0);
    CHECK(std::strcmp(creator->getPluginVersion(), "1") == 0);
    CHECK(std::strcmp(creator->getPluginNamespace(), "") == 0);
    PluginFieldCollection const* names = creator->getFieldNames();
    CHECK(names->nbFields == 3);
    CHECK(std::strcmp(names->fields[0].name, "scale") == 0 && std::strcmp(names->fields[1].name, "gk_normalizer") == 0 &&
          std::strcmp(names->fields[2].name, "rms_eps") == 0);

    const float scale = 0.176776695f, norm = 16.0f;
    const double eps = 1e-5;                                  // a FLOAT64 field must be accepted too
    PluginField in_fields[3] = {{"rms_eps", &eps, PluginFieldType::kFLOAT64, 1},
                                {"scale", &scale, PluginFieldType::kFLOAT32, 1},
                                {"gk_normalizer", &norm, PluginFieldType::kFLOAT32, 1}};
    PluginFieldCollection fc{3, in_fields};
    IPluginV3* plugin = creator->createPlugin("gla", &fc, TensorRTPhase::kBUILD);
    CHECK(plugin != nullptr);
    auto* core = static_cast<IPluginV3OneCore*>(plugin->getCapabilityInterface(PluginCapabilityType::kCORE));
    auto* build = static_cast<IPluginV3OneBuild*>(plugin->getCapabilityInterface(PluginCapabilityType::kBUILD));
    auto* run = static_cast<IPluginV3OneRuntime*>(plugin->getCapabilityInterface(PluginCapabilityType::kRUNTIME));
    CHECK(std::strcmp(core->getPluginName(), "GatedLinearAttention") == 0);
    CHECK(build->getNbOutputs() == 1);
    PluginFieldCollection const* ser = run->getFieldsToSerialize();
    CHECK(ser->nbFields == 3);
    CHECK(*static_cast<float const*>(ser->fields[0].data) == scale);
    CHECK(*static_cast<float const*>(ser->fields[1].data) == norm);
    CHECK(*static_cast<float const*>(ser->fields[2].data) == static_cast<float>(eps));

    DynamicPluginTensorDesc io[7] = {desc(1, 1600, 3, 32), desc(1, 1600, 3, 32), desc(1, 1600, 3, 64), desc(1, 1600, 3, 32),
                                     desc(1, 1600, 3, 64), desc(64, 1, 1, 1), desc(1, 1600, 3, 64)};
    CHECK(build->configurePlugin(io, 6, io + 6, 1) == 0);
    CHECK(build->configurePlugin(io, 5, io + 6, 1) == -1);
    for (int pos = 0; pos < 7; ++pos) CHECK(build->supportsFormatCombination(pos, io, 6, 1));
    DynamicPluginTensorDesc f32 = desc(1, 1600, 3, 32, DataType::kFLOAT);
    CHECK(!build->supportsFormatCombination(0, &f32, 1, 0));
    DataType in_types[6] = {DataType::kHALF, DataType::kHALF, DataType::kHALF, DataType::kHALF, DataType::kHALF, DataType::kHALF};
    DataType out_type = DataType::kFLOAT;
    CHECK(build->getOutputDataTypes(&out_type, 1, in_types, 6) == 0 && out_type == DataType::kHALF);
    const size_t ws = build->getWorkspaceSize(io, 6, io + 6, 1);
    CHECK(ws == gla_b200_workspace_bytes(1, 1600, 3, 32, 64) + 256);
    DynamicPluginTensorDesc k64[3] = {desc(4, 6400, 12, 64), desc(4, 6400, 12, 64), desc(4, 6400, 12, 64)};
    CHECK(build->getWorkspaceSize(k64, 3, nullptr, 0) == gla_b200_workspace_bytes(4, 6400, 12, 64, 64) + 256);
    DynamicPluginTensorDesc bad[3] = {desc(1, 64, 1, 48), desc(1, 64, 1, 48), desc(1, 64, 1, 64)};
    CHECK(build->getWorkspaceSize(bad, 3, nullptr, 0) == 0);             // K = 48 is not served

    // enqueue refuses what it cannot run, without touching a device
    PluginTensorDesc in_desc[6];
    for (int i = 0; i < 6; ++i) in_desc[i] = io[i].desc;
    CHECK(run->onShapeChange(in_desc, 6, &io[6].desc, 1) == 0);
    void const* ins[6] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
    void* outs[1] = {nullptr};
    CHECK(run->enqueue(in_desc, &io[6].desc, ins, outs, nullptr, nullptr) == -1);     // no workspace

    IPluginV3* copy = plugin->clone();
    auto* run2 = static_cast<IPluginV3OneRuntime*>(copy->getCapabilityInterface(PluginCapabilityType::kRUNTIME));
    CHECK(*static_cast<float const*>(run2->getFieldsToSerialize()->fields[0].data) == scale);
    IPluginV3* attached = run->attachToContext(nullptr);
    CHECK(attached != nullptr && attached != plugin);
    delete attached;
    delete copy;
    delete plugin;
    std::printf("%d failure(s)\n", failures);
    return failures;
}
