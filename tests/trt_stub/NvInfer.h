// Stand-in for TensorRT's NvInfer.h: just enough declarations of the public plugin interfaces (IPluginV3 and its
// build / runtime / core capabilities, IPluginCreatorV3One, the descriptor structs) for
// gtr_b200/csrc/gla_plugin_b200.cu to compile and for its logic to be exercised on a machine that has no TensorRT.
// Test infrastructure only; not an implementation of TensorRT and never installed.
#pragma once
#include <cstddef>
#include <cstdint>
#include <new>

struct CUstream_st;
typedef CUstream_st* cudaStream_t;

namespace nvinfer1 {

enum class DataType : int32_t { kFLOAT = 0, kHALF = 1, kINT8 = 2, kINT32 = 3 };
enum class TensorFormat : int32_t { kLINEAR = 0, kCHW2 = 1 };
enum class PluginFieldType : int32_t { kFLOAT16 = 0, kFLOAT32 = 1, kFLOAT64 = 2, kINT8 = 3, kINT16 = 4, kINT32 = 5 };
enum class PluginCapabilityType : int32_t { kCORE = 0, kBUILD = 1, kRUNTIME = 2 };
enum class TensorRTPhase : int32_t { kBUILD = 0, kRUNTIME = 1 };

struct Dims {
    static constexpr int32_t MAX_DIMS = 8;
    int32_t nbDims;
    int64_t d[MAX_DIMS];
};
struct PluginTensorDesc {
    Dims dims;
    DataType type;
    TensorFormat format;
    float scale;
};
struct DynamicPluginTensorDesc {
    PluginTensorDesc desc;
    Dims min, opt, max;
};
class IDimensionExpr;
struct DimsExprs {
    int32_t nbDims;
    IDimensionExpr const* d[Dims::MAX_DIMS];
};
class IExprBuilder {};
class IPluginResourceContext {};

struct PluginField {
    char const* name;
    void const* data;
    PluginFieldType type;
    int32_t length;
};
struct PluginFieldCollection {
    int32_t nbFields;
    PluginField const* fields;
};

class IPluginCapability {
public:
    virtual ~IPluginCapability() = default;
};
class IPluginV3 {
public:
    virtual ~IPluginV3() = default;
    virtual IPluginCapability* getCapabilityInterface(PluginCapabilityType type) noexcept = 0;
    virtual IPluginV3* clone() noexcept = 0;
};
class IPluginV3OneCore : public IPluginCapability {
public:
    virtual char const* getPluginName() const noexcept = 0;
    virtual char const* getPluginVersion() const noexcept = 0;
    virtual char const* getPluginNamespace() const noexcept = 0;
};
class IPluginV3OneBuild : public IPluginCapability {
public:
    virtual int32_t configurePlugin(DynamicPluginTensorDesc const* in, int32_t nbInputs, DynamicPluginTensorDesc const* out,
                                    int32_t nbOutputs) noexcept = 0;
    virtual int32_t getOutputDataTypes(DataType* outputTypes, int32_t nbOutputs, DataType const* inputTypes,
                                       int32_t nbInputs) const noexcept = 0;
    virtual int32_t getOutputShapes(DimsExprs const* inputs, int32_t nbInputs, DimsExprs const* shapeInputs,
                                    int32_t nbShapeInputs, DimsExprs* outputs, int32_t nbOutputs,
                                    IExprBuilder& exprBuilder) noexcept = 0;
    virtual bool supportsFormatCombination(int32_t pos, DynamicPluginTensorDesc const* inOut, int32_t nbInputs,
                                           int32_t nbOutputs) noexcept = 0;
    virtual int32_t getNbOutputs() const noexcept = 0;
    virtual size_t getWorkspaceSize(DynamicPluginTensorDesc const* inputs, int32_t nbInputs,
                                    DynamicPluginTensorDesc const* outputs, int32_t nbOutputs) const noexcept = 0;
};
class IPluginV3OneRuntime : public IPluginCapability {
public:
    virtual int32_t onShapeChange(PluginTensorDesc const* in, int32_t nbInputs, PluginTensorDesc const* out,
                                  int32_t nbOutputs) noexcept = 0;
    virtual int32_t enqueue(PluginTensorDesc const* inputDesc, PluginTensorDesc const* outputDesc, void const* const* inputs,
                            void* const* outputs, void* workspace, cudaStream_t stream) noexcept = 0;
    virtual IPluginV3* attachToContext(IPluginResourceContext* context) noexcept = 0;
    virtual PluginFieldCollection const* getFieldsToSerialize() noexcept = 0;
};
class IPluginCreatorV3One {
public:
    virtual ~IPluginCreatorV3One() = default;
    virtual IPluginV3* createPlugin(char const* name, PluginFieldCollection const* fc, TensorRTPhase phase) noexcept = 0;
    virtual PluginFieldCollection const* getFieldNames() noexcept = 0;
    virtual char const* getPluginName() const noexcept = 0;
    virtual char const* getPluginVersion() const noexcept = 0;
    virtual char const* getPluginNamespace() const noexcept = 0;
};

}  // namespace nvinfer1

#define REGISTER_TENSORRT_PLUGIN(name) static name pluginRegistrar##name {}
