// Host-side mirror of the reference's plugins: the four of the sparse front end, ZeroPad2d, and the two
// detection post-processing plugins (GenerateAnchorDecode, FilterBoxByScore).
//
// Same class names, creator field names, member-function names, tensor orders, return conventions and
// serialised byte layouts as the reference's TensorRT plugins; the bodies call the C ABI of sessd.h
// instead of the reference's kernels. TensorRT's headers are not required: the small structs of
// sessd_plugins.h stand in for PluginTensorDesc / PluginField, and output dimensions are returned as
// plain integers instead of IExprBuilder expressions. A TensorRT shim deriving from
// IPluginV2DynamicExt only has to forward each virtual to the member of the same name.
#pragma once

#include <cstdint>
#include <string>
#include <vector>

#include "sessd.h"
#include "sessd_plugins.h"

namespace sessd {
namespace plugin {

using TensorDesc = sessd_tensor_desc;
using Field = sessd_plugin_field;

// Members every plugin offers (the subset of IPluginV2DynamicExt the reference implements,
// e.g. submConv3dlayer.h:34-62).
class PluginBase {
public:
    virtual ~PluginBase() {}
    virtual PluginBase* clone() const = 0;
    virtual int getOutputDimensions(int outputIndex, const TensorDesc* inputs, int nbInputs, TensorDesc* out) const = 0;
    virtual bool supportsFormatCombination(int pos, const TensorDesc* inOut, int nbInputs, int nbOutputs) const = 0;
    virtual void configurePlugin(const TensorDesc* in, int nbInputs, const TensorDesc* out, int nbOutputs) = 0;
    virtual size_t getWorkspaceSize(const TensorDesc* inputs, int nbInputs, const TensorDesc* outputs,
                                    int nbOutputs) const = 0;
    virtual int enqueue(const TensorDesc* inputDesc, const TensorDesc* outputDesc, const void* const* inputs,
                        void* const* outputs, void* workspace, void* stream) = 0;
    virtual int getOutputDataType(int index, const int32_t* inputTypes, int nbInputs) const = 0;
    virtual const char* getPluginType() const = 0;
    virtual const char* getPluginVersion() const { return "1"; }
    virtual int getNbOutputs() const = 0;
    virtual int initialize() { return 0; }
    virtual void terminate() {}
    virtual size_t getSerializationSize() const = 0;
    virtual void serialize(void* buffer) const = 0;
    virtual void destroy() { delete this; }
    void setPluginNamespace(const char* ns) { mNamespace = ns ? ns : ""; }
    const char* getPluginNamespace() const { return mNamespace.c_str(); }

protected:
    std::string mNamespace;
};

// voxelGenerator.h:19-110. Inputs {points f32 [B,P,4], points_size i32 [B]};
// outputs {voxels [B,maxV,4], coors i32 [B,maxV,4], voxel_num i32 [B]}.
class VoxelGeneratorPlugin : public PluginBase {
public:
    VoxelGeneratorPlugin(int max_voxels, int max_points, int voxel_features, float x_min, float x_max, float y_min,
                         float y_max, float z_min, float z_max, float voxel_x, float voxel_y, float voxel_z);
    VoxelGeneratorPlugin(const void* data, size_t length);
    PluginBase* clone() const override;
    int getOutputDimensions(int outputIndex, const TensorDesc* inputs, int nbInputs, TensorDesc* out) const override;
    bool supportsFormatCombination(int pos, const TensorDesc* inOut, int nbInputs, int nbOutputs) const override;
    void configurePlugin(const TensorDesc* in, int nbInputs, const TensorDesc* out, int nbOutputs) override;
    size_t getWorkspaceSize(const TensorDesc* inputs, int nbInputs, const TensorDesc* outputs, int nbOutputs) const override;
    int enqueue(const TensorDesc* inputDesc, const TensorDesc* outputDesc, const void* const* inputs,
                void* const* outputs, void* workspace, void* stream) override;
    int getOutputDataType(int index, const int32_t* inputTypes, int nbInputs) const override;
    const char* getPluginType() const override { return "VoxelGeneratorPlugin"; }
    int getNbOutputs() const override { return 3; }
    size_t getSerializationSize() const override { return sizeof(sessd_voxel_params); }
    void serialize(void* buffer) const override;

private:
    sessd_voxel_params p_;  // field for field the reference's members and serialisation order
};

// submConv3dlayer.h:19-121 and sparseConv3dlayer.h:18-126 share everything but the integer lists.
class ConvPluginBase : public PluginBase {
public:
    ~ConvPluginBase() override;
    bool supportsFormatCombination(int pos, const TensorDesc* inOut, int nbInputs, int nbOutputs) const override;
    void configurePlugin(const TensorDesc*, int, const TensorDesc*, int) override {}
    size_t getWorkspaceSize(const TensorDesc* inputs, int nbInputs, const TensorDesc* outputs, int nbOutputs) const override;
    int enqueue(const TensorDesc* inputDesc, const TensorDesc* outputDesc, const void* const* inputs,
                void* const* outputs, void* workspace, void* stream) override;
    int getOutputDataType(int index, const int32_t* inputTypes, int nbInputs) const override;
    void terminate() override;

protected:
    ConvPluginBase(const sessd_conv_params& p, const float* weights, int weights_size);
    int ensureWeights(int dtype);   // uploads on first use per data type (the reference uploads in its constructor)
    sessd_conv_params p_;
    std::vector<float> weights_;    // host copy, as the reference keeps (weights_data_)
    sessd_conv_weights* dev_[2];    // per feature data type
};

class SubmConv3dLayerPlugin : public ConvPluginBase {
public:
    SubmConv3dLayerPlugin(int in_channel, int out_channel, int max_voxels, int feature_num, int out_shape_x,
                          int out_shape_y, int out_shape_z, int spatial_shape_x, int spatial_shape_y,
                          int spatial_shape_z, int ksize, int stride, int padding, int dilation, int out_padding,
                          int weights_size, const float* weights);
    SubmConv3dLayerPlugin(const void* data, size_t length);
    PluginBase* clone() const override;
    int getOutputDimensions(int outputIndex, const TensorDesc* inputs, int nbInputs, TensorDesc* out) const override;
    const char* getPluginType() const override { return "SubmConv3dLayerPlugin"; }
    int getNbOutputs() const override { return 1; }
    size_t getSerializationSize() const override;
    void serialize(void* buffer) const override;

private:
    int stride_;   // serialised but unused by a submanifold layer
};

class SparseConv3dLayerPlugin : public ConvPluginBase {
public:
    SparseConv3dLayerPlugin(int in_channel, int out_channel, int max_voxels, int feature_num, int out_shape_x,
                            int out_shape_y, int out_shape_z, int spatial_shape_x, int spatial_shape_y,
                            int spatial_shape_z, int ksize0, int ksize1, int ksize2, int stride0, int stride1,
                            int stride2, int padding0, int padding1, int padding2, int dilation, int out_padding,
                            int weights_size, const float* weights);
    SparseConv3dLayerPlugin(const void* data, size_t length);
    PluginBase* clone() const override;
    int getOutputDimensions(int outputIndex, const TensorDesc* inputs, int nbInputs, TensorDesc* out) const override;
    const char* getPluginType() const override { return "SparseConv3dLayerPlugin"; }
    int getNbOutputs() const override { return 3; }
    size_t getSerializationSize() const override;
    void serialize(void* buffer) const override;
};

// sparse2Dense.h:18-86. Inputs {features, coors, voxel_num}; output {dense [B, C*D, H, W]}.
class Sparse2DensePlugin : public PluginBase {
public:
    Sparse2DensePlugin(int feature_map_size_x, int feature_map_size_y, int feature_map_size_z, int feature_map_channel);
    Sparse2DensePlugin(const void* data, size_t length);
    PluginBase* clone() const override;
    int getOutputDimensions(int outputIndex, const TensorDesc* inputs, int nbInputs, TensorDesc* out) const override;
    bool supportsFormatCombination(int pos, const TensorDesc* inOut, int nbInputs, int nbOutputs) const override;
    void configurePlugin(const TensorDesc*, int, const TensorDesc*, int) override {}
    size_t getWorkspaceSize(const TensorDesc*, int, const TensorDesc*, int) const override { return 0; }
    int enqueue(const TensorDesc* inputDesc, const TensorDesc* outputDesc, const void* const* inputs,
                void* const* outputs, void* workspace, void* stream) override;
    int getOutputDataType(int index, const int32_t* inputTypes, int nbInputs) const override;
    const char* getPluginType() const override { return "Sparse2DensePlugin"; }
    int getNbOutputs() const override { return 1; }
    size_t getSerializationSize() const override { return sizeof(sessd_s2d_params); }
    void serialize(void* buffer) const override;

private:
    sessd_s2d_params p_;
};

// zeroPad2d.h:18-87. Input {map [B, C, H, W]}; output {map [B, C, top+H+bottom, left+W+right]}.
class ZeroPad2dPlugin : public PluginBase {
public:
    ZeroPad2dPlugin(int zero_padding_2d_top, int zero_padding_2d_bottom, int zero_padding_2d_left,
                    int zero_padding_2d_right);
    ZeroPad2dPlugin(const void* data, size_t length);
    PluginBase* clone() const override;
    int getOutputDimensions(int outputIndex, const TensorDesc* inputs, int nbInputs, TensorDesc* out) const override;
    bool supportsFormatCombination(int pos, const TensorDesc* inOut, int nbInputs, int nbOutputs) const override;
    void configurePlugin(const TensorDesc*, int, const TensorDesc*, int) override {}
    size_t getWorkspaceSize(const TensorDesc*, int, const TensorDesc*, int) const override { return 0; }
    int enqueue(const TensorDesc* inputDesc, const TensorDesc* outputDesc, const void* const* inputs,
                void* const* outputs, void* workspace, void* stream) override;
    int getOutputDataType(int index, const int32_t* inputTypes, int nbInputs) const override;
    const char* getPluginType() const override { return "ZeroPad2dPlugin"; }
    int getNbOutputs() const override { return 1; }
    size_t getSerializationSize() const override { return sizeof(sessd_pad2d_params); }
    void serialize(void* buffer) const override;

private:
    sessd_pad2d_params p_;
};

// generateAnchorDecode.h:19-106. Input {box_preds f32 [B, N, 7]}; output {boxes f32 [B, N, 7]}.
class GenerateAnchorDecodePlugin : public PluginBase {
public:
    GenerateAnchorDecodePlugin(float min_x_range, float max_x_range, float min_y_range, float max_y_range,
                               float min_z_range, float max_z_range, int feature_map_height, int feature_map_width,
                               float car_length, float car_width, float car_height, float direction_angle_0,
                               float direction_angle_1, int direction_angle_num);
    GenerateAnchorDecodePlugin(const void* data, size_t length);
    PluginBase* clone() const override;
    int getOutputDimensions(int outputIndex, const TensorDesc* inputs, int nbInputs, TensorDesc* out) const override;
    bool supportsFormatCombination(int pos, const TensorDesc* inOut, int nbInputs, int nbOutputs) const override;
    void configurePlugin(const TensorDesc*, int, const TensorDesc*, int) override {}
    size_t getWorkspaceSize(const TensorDesc*, int, const TensorDesc*, int) const override { return 0; }
    int enqueue(const TensorDesc* inputDesc, const TensorDesc* outputDesc, const void* const* inputs,
                void* const* outputs, void* workspace, void* stream) override;
    int getOutputDataType(int index, const int32_t* inputTypes, int nbInputs) const override;
    const char* getPluginType() const override { return "GenerateAnchorDecodePlugin"; }
    int getNbOutputs() const override { return 1; }
    size_t getSerializationSize() const override { return sizeof(sessd_anchor_params); }
    void serialize(void* buffer) const override;
    const sessd_anchor_params& params() const { return p_; }

private:
    sessd_anchor_params p_;
};

// filterBoxByScore.h:18-90. Inputs {boxes [B, N, 7], cls_preds [B, N, 1], iou_preds [B, N, 1], dir_preds
// [B, N, 2]}; outputs {box [B, max_box, 9], score [B, max_box], iou [B, max_box, 1], direction
// [B, max_box, 1], valid_line_num i32 [B, 1]}.
class FilterBoxByScorePlugin : public PluginBase {
public:
    FilterBoxByScorePlugin(int feature_map_height, int feature_map_width, int direction_angle_num, int max_box_num,
                           float score_threshold, float direction_offset);
    FilterBoxByScorePlugin(const void* data, size_t length);
    PluginBase* clone() const override;
    int getOutputDimensions(int outputIndex, const TensorDesc* inputs, int nbInputs, TensorDesc* out) const override;
    bool supportsFormatCombination(int pos, const TensorDesc* inOut, int nbInputs, int nbOutputs) const override;
    void configurePlugin(const TensorDesc*, int, const TensorDesc*, int) override {}
    size_t getWorkspaceSize(const TensorDesc* inputs, int nbInputs, const TensorDesc* outputs, int nbOutputs) const override;
    int enqueue(const TensorDesc* inputDesc, const TensorDesc* outputDesc, const void* const* inputs,
                void* const* outputs, void* workspace, void* stream) override;
    int getOutputDataType(int index, const int32_t* inputTypes, int nbInputs) const override;
    const char* getPluginType() const override { return "FilterBoxByScorePlugin"; }
    int getNbOutputs() const override { return 5; }
    size_t getSerializationSize() const override { return sizeof(sessd_filter_params); }
    void serialize(void* buffer) const override;

private:
    sessd_filter_params p_;
};

// IPluginCreator mirror: field names as the reference advertises them (e.g. submConv3dlayer.cu:737-748).
class PluginCreator {
public:
    virtual ~PluginCreator() {}
    virtual const char* getPluginName() const = 0;
    virtual const char* getPluginVersion() const { return "1"; }
    virtual const std::vector<std::string>& getFieldNames() const = 0;
    virtual PluginBase* createPlugin(const char* name, const Field* fields, int nbFields) const = 0;
    virtual PluginBase* deserializePlugin(const char* name, const void* serialData, size_t serialLength) const = 0;
};

// Registry lookup by (name, "1"), as getPluginRegistry()->getPluginCreator does in the reference
// (se-ssd-ai-trt.cpp:339, :707, :911, :571).
const PluginCreator* getPluginCreator(const char* name, const char* version);

}  // namespace plugin
}  // namespace sessd
