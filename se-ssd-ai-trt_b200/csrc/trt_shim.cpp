// TensorRT face of the plugin mirrors: IPluginV2DynamicExt + IPluginCreator + REGISTER_TENSORRT_PLUGIN.
//
// The reference's seven plugins derive from nvinfer1::IPluginV2DynamicExt and register a creator each
// (voxelGenerator.h:17-111, submConv3dlayer.h:19-121, sparseConv3dlayer.h:18-126, sparse2Dense.h:18-86,
// zeroPad2d.h:18-87, generateAnchorDecode.h:19-106, filterBoxByScore.h:18-90). The classes of plugins.h carry
// the same names, members, creator fields and serialised bytes without needing TensorRT; this file puts the
// TensorRT base classes on top of them: every virtual forwards to the member of the same name, tensor
// descriptors and plugin fields are converted one to one. With these creators registered, a network built by
// the reference's own code (se-ssd-ai-trt.cpp:339, :571, :707, :911 look the creators up by name and version)
// and an engine it serialised run on this library unchanged.
//
// The whole file is empty unless TensorRT's NvInferPlugin.h can be found when it is compiled; the build script
// adds it to the library (and links nvinfer) only then. NVIDIA's headers are neither copied nor restated here.
#if defined(__has_include)
#if __has_include(<NvInferPlugin.h>)
#define SESSD_HAVE_TENSORRT 1
#endif
#endif

#ifdef SESSD_HAVE_TENSORRT

#include <NvInferPlugin.h>
#include <cuda_runtime_api.h>

#include <cstring>
#include <mutex>
#include <string>
#include <vector>

#include "plugins.h"

namespace sessd {
namespace trt {

using nvinfer1::DataType;
using nvinfer1::DimsExprs;
using nvinfer1::DynamicPluginTensorDesc;
using nvinfer1::IExprBuilder;
using nvinfer1::IPluginV2;
using nvinfer1::IPluginV2DynamicExt;
using nvinfer1::PluginField;
using nvinfer1::PluginFieldCollection;
using nvinfer1::PluginTensorDesc;

namespace {

plugin::TensorDesc to_desc(const PluginTensorDesc& d) {
    plugin::TensorDesc t{};
    t.nb_dims = d.dims.nbDims;
    for (int i = 0; i < d.dims.nbDims && i < 8; ++i) t.d[i] = d.dims.d[i];
    t.dtype = static_cast<int32_t>(d.type);
    t.format = static_cast<int32_t>(d.format) == static_cast<int32_t>(nvinfer1::TensorFormat::kLINEAR) ? 0 : 1;
    return t;
}

std::vector<plugin::TensorDesc> to_descs(const PluginTensorDesc* d, int n) {
    std::vector<plugin::TensorDesc> v(n > 0 ? n : 0);
    for (int i = 0; i < n; ++i) v[i] = to_desc(d[i]);
    return v;
}

}  // namespace

// One class serves all seven plugins: what differs between them lives in the mirror object it owns.
class Plugin : public IPluginV2DynamicExt {
public:
    explicit Plugin(plugin::PluginBase* impl) : impl_(impl) {}
    ~Plugin() override { if (impl_) impl_->destroy(); }

    IPluginV2DynamicExt* clone() const noexcept override {
        plugin::PluginBase* c = impl_->clone();
        if (!c) return nullptr;
        Plugin* p = new Plugin(c);
        p->setPluginNamespace(impl_->getPluginNamespace());
        return p;
    }

    // The mirrors compute output shapes from concrete input shapes. Dimensions that are build-time constants are
    // passed as such; a dynamic batch dimension (dimension 0) is carried through as the expression it is.
    DimsExprs getOutputDimensions(int32_t outputIndex, const DimsExprs* inputs, int32_t nbInputs,
                                  IExprBuilder& exprBuilder) noexcept override {
        std::vector<plugin::TensorDesc> in(nbInputs > 0 ? nbInputs : 0);
        for (int i = 0; i < nbInputs; ++i) {
            in[i].nb_dims = inputs[i].nbDims;
            for (int j = 0; j < inputs[i].nbDims && j < 8; ++j)
                in[i].d[j] = inputs[i].d[j]->isConstant() ? inputs[i].d[j]->getConstantValue() : 1;
        }
        plugin::TensorDesc out{};
        DimsExprs r{};
        if (impl_->getOutputDimensions(outputIndex, in.data(), nbInputs, &out) != 0) return r;
        r.nbDims = out.nb_dims;
        for (int j = 0; j < out.nb_dims; ++j) r.d[j] = exprBuilder.constant(out.d[j]);
        if (nbInputs > 0 && inputs[0].nbDims > 0 && r.nbDims > 0 && !inputs[0].d[0]->isConstant()) r.d[0] = inputs[0].d[0];
        return r;
    }

    bool supportsFormatCombination(int32_t pos, const PluginTensorDesc* inOut, int32_t nbInputs,
                                   int32_t nbOutputs) noexcept override {
        const std::vector<plugin::TensorDesc> d = to_descs(inOut, nbInputs + nbOutputs);
        return impl_->supportsFormatCombination(pos, d.data(), nbInputs, nbOutputs);
    }

    void configurePlugin(const DynamicPluginTensorDesc* in, int32_t nbInputs, const DynamicPluginTensorDesc* out,
                         int32_t nbOutputs) noexcept override {
        std::vector<plugin::TensorDesc> i(nbInputs > 0 ? nbInputs : 0), o(nbOutputs > 0 ? nbOutputs : 0);
        for (int k = 0; k < nbInputs; ++k) i[k] = to_desc(in[k].desc);
        for (int k = 0; k < nbOutputs; ++k) o[k] = to_desc(out[k].desc);
        impl_->configurePlugin(i.data(), nbInputs, o.data(), nbOutputs);
    }

    size_t getWorkspaceSize(const PluginTensorDesc* inputs, int32_t nbInputs, const PluginTensorDesc* outputs,
                            int32_t nbOutputs) const noexcept override {
        const std::vector<plugin::TensorDesc> i = to_descs(inputs, nbInputs), o = to_descs(outputs, nbOutputs);
        return impl_->getWorkspaceSize(i.data(), nbInputs, o.data(), nbOutputs);
    }

    // 0 = ok, as the reference returns; any library error becomes a non-zero return instead of the
    // reference's abort() (voxelGenerator.cu:8-19).
    int32_t enqueue(const PluginTensorDesc* inputDesc, const PluginTensorDesc* outputDesc, const void* const* inputs,
                    void* const* outputs, void* workspace, cudaStream_t stream) noexcept override {
        // descriptor counts are not passed by TensorRT: the mirrors know how many tensors they take
        plugin::TensorDesc in[8], out[8];
        const int n_in = inputCount(), n_out = impl_->getNbOutputs();
        for (int k = 0; k < n_in && k < 8; ++k) in[k] = to_desc(inputDesc[k]);
        for (int k = 0; k < n_out && k < 8; ++k) out[k] = to_desc(outputDesc[k]);
        return impl_->enqueue(in, out, inputs, outputs, workspace, static_cast<void*>(stream));
    }

    DataType getOutputDataType(int32_t index, const DataType* inputTypes, int32_t nbInputs) const noexcept override {
        int32_t t[8] = {0};
        for (int k = 0; k < nbInputs && k < 8; ++k) t[k] = static_cast<int32_t>(inputTypes[k]);
        return static_cast<DataType>(impl_->getOutputDataType(index, t, nbInputs));
    }

    const char* getPluginType() const noexcept override { return impl_->getPluginType(); }
    const char* getPluginVersion() const noexcept override { return impl_->getPluginVersion(); }
    int32_t getNbOutputs() const noexcept override { return impl_->getNbOutputs(); }
    int32_t initialize() noexcept override { return impl_->initialize(); }
    void terminate() noexcept override { impl_->terminate(); }
    size_t getSerializationSize() const noexcept override { return impl_->getSerializationSize(); }
    void serialize(void* buffer) const noexcept override { impl_->serialize(buffer); }
    void destroy() noexcept override { delete this; }
    void setPluginNamespace(const char* ns) noexcept override { impl_->setPluginNamespace(ns); }
    const char* getPluginNamespace() const noexcept override { return impl_->getPluginNamespace(); }

private:
    // number of input tensors of the wrapped plugin (voxelGenerator.cu:161-226 and the sibling files)
    int inputCount() const {
        const std::string t = impl_->getPluginType();
        if (t == "VoxelGeneratorPlugin") return 2;
        if (t == "ZeroPad2dPlugin" || t == "GenerateAnchorDecodePlugin") return 1;
        if (t == "FilterBoxByScorePlugin") return 4;
        return 3;   // the two convolutions and Sparse2Dense: features, coors, voxel_num
    }
    plugin::PluginBase* impl_;
};

// IPluginCreator over the mirror creator of the same name.
template <int ID>
class Creator : public nvinfer1::IPluginCreator {
public:
    Creator() {
        const plugin::PluginCreator* c = plugin::getPluginCreator(name(), "1");
        if (c)
            for (const std::string& f : c->getFieldNames())
                // the reference declares every field as kFLOAT32 with length 1 whatever it holds
                // (voxelGenerator.cu:624-628); only the names matter to createPlugin, which reads by pointer
                fields_.push_back(PluginField(f.c_str(), nullptr, nvinfer1::PluginFieldType::kFLOAT32, 1));
        fc_.nbFields = static_cast<int32_t>(fields_.size());
        fc_.fields = fields_.data();
    }
    static const char* name();
    const char* getPluginName() const noexcept override { return name(); }
    const char* getPluginVersion() const noexcept override { return "1"; }
    const PluginFieldCollection* getFieldNames() noexcept override { return &fc_; }

    IPluginV2* createPlugin(const char* layerName, const PluginFieldCollection* fc) noexcept override {
        const plugin::PluginCreator* c = plugin::getPluginCreator(name(), "1");
        if (!c || !fc) return nullptr;
        std::vector<plugin::Field> f(fc->nbFields > 0 ? fc->nbFields : 0);
        for (int i = 0; i < fc->nbFields; ++i)
            f[i] = plugin::Field{fc->fields[i].name, fc->fields[i].data, static_cast<int32_t>(fc->fields[i].type),
                                 fc->fields[i].length};
        plugin::PluginBase* p = c->createPlugin(layerName, f.data(), fc->nbFields);
        if (!p) return nullptr;
        Plugin* out = new Plugin(p);
        out->setPluginNamespace(ns_.c_str());
        return out;
    }

    IPluginV2* deserializePlugin(const char* layerName, const void* serialData, size_t serialLength) noexcept override {
        const plugin::PluginCreator* c = plugin::getPluginCreator(name(), "1");
        if (!c) return nullptr;
        plugin::PluginBase* p = c->deserializePlugin(layerName, serialData, serialLength);
        if (!p) return nullptr;
        Plugin* out = new Plugin(p);
        out->setPluginNamespace(ns_.c_str());
        return out;
    }

    void setPluginNamespace(const char* ns) noexcept override { ns_ = ns ? ns : ""; }
    const char* getPluginNamespace() const noexcept override { return ns_.c_str(); }

private:
    std::vector<PluginField> fields_;
    PluginFieldCollection fc_{};
    std::string ns_;
};

template <> const char* Creator<0>::name() { return "VoxelGeneratorPlugin"; }
template <> const char* Creator<1>::name() { return "SubmConv3dLayerPlugin"; }
template <> const char* Creator<2>::name() { return "SparseConv3dLayerPlugin"; }
template <> const char* Creator<3>::name() { return "Sparse2DensePlugin"; }
template <> const char* Creator<4>::name() { return "ZeroPad2dPlugin"; }
template <> const char* Creator<5>::name() { return "GenerateAnchorDecodePlugin"; }
template <> const char* Creator<6>::name() { return "FilterBoxByScorePlugin"; }

using VoxelGeneratorPluginCreator = Creator<0>;
using SubmConv3dLayerPluginCreator = Creator<1>;
using SparseConv3dLayerPluginCreator = Creator<2>;
using Sparse2DensePluginCreator = Creator<3>;
using ZeroPad2dPluginCreator = Creator<4>;
using GenerateAnchorDecodePluginCreator = Creator<5>;
using FilterBoxByScorePluginCreator = Creator<6>;

// the same registrations the reference makes at the end of each plugin header (e.g. voxelGenerator.h:111); the macro
// pastes the class name into a variable name, hence the unqualified aliases
REGISTER_TENSORRT_PLUGIN(VoxelGeneratorPluginCreator);
REGISTER_TENSORRT_PLUGIN(SubmConv3dLayerPluginCreator);
REGISTER_TENSORRT_PLUGIN(SparseConv3dLayerPluginCreator);
REGISTER_TENSORRT_PLUGIN(Sparse2DensePluginCreator);
REGISTER_TENSORRT_PLUGIN(ZeroPad2dPluginCreator);
REGISTER_TENSORRT_PLUGIN(GenerateAnchorDecodePluginCreator);
REGISTER_TENSORRT_PLUGIN(FilterBoxByScorePluginCreator);

}  // namespace trt
}  // namespace sessd

extern "C" int sessd_tensorrt_shim_present(void) { return 1; }

#else  // no TensorRT headers where this file is compiled

extern "C" int sessd_tensorrt_shim_present(void) { return 0; }

#endif
