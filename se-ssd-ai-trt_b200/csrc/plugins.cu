// Implementation of the plugin mirror (plugins.h) and of its C view (sessd_plugins.h).
#include "plugins.h"

#include <cstring>

namespace sessd {
namespace plugin {

namespace {

template <typename T>
void put(char*& d, const T& v) {
    std::memcpy(d, &v, sizeof(T));
    d += sizeof(T);
}
template <typename T>
T get(const char*& d) {
    T v;
    std::memcpy(&v, d, sizeof(T));
    d += sizeof(T);
    return v;
}

TensorDesc make_desc(std::initializer_list<int> dims, int dtype) {
    TensorDesc t{};
    t.nb_dims = (int)dims.size();
    int i = 0;
    for (int v : dims) t.d[i++] = v;
    t.dtype = dtype;
    t.format = 0;
    return t;
}

int feature_dtype(const TensorDesc& t) { return t.dtype == SESSD_DT_HALF ? SESSD_F16 : SESSD_F32; }
bool is_feature_type(const TensorDesc& t) {
    return (t.dtype == SESSD_DT_FLOAT || t.dtype == SESSD_DT_HALF) && t.format == 0;
}
bool is_int32(const TensorDesc& t) { return t.dtype == SESSD_DT_INT32 && t.format == 0; }

}  // namespace

// ---------------------------------------------------------------- VoxelGeneratorPlugin

VoxelGeneratorPlugin::VoxelGeneratorPlugin(int max_voxels, int max_points, int voxel_features, float x_min, float x_max,
                                           float y_min, float y_max, float z_min, float z_max, float voxel_x,
                                           float voxel_y, float voxel_z) {
    // argument order of the reference constructor (voxelGenerator.cu:105-115); max_points is the
    // per-voxel point capacity (pointNum_)
    p_ = sessd_voxel_params{max_voxels, max_points, voxel_features, x_min, x_max, y_min, y_max, z_min, z_max,
                            voxel_x,    voxel_y,    voxel_z,        0,     0,     0,     0};
}

VoxelGeneratorPlugin::VoxelGeneratorPlugin(const void* data, size_t length) {
    std::memset(&p_, 0, sizeof(p_));
    if (data && length >= sizeof(p_)) std::memcpy(&p_, data, sizeof(p_));   // voxelGenerator.cu:131-150
}

PluginBase* VoxelGeneratorPlugin::clone() const {
    auto* c = new VoxelGeneratorPlugin(*this);
    return c;
}

int VoxelGeneratorPlugin::getOutputDimensions(int outputIndex, const TensorDesc* inputs, int nbInputs,
                                              TensorDesc* out) const {
    if (!inputs || nbInputs < 1 || !out) return -1;
    const int batch = inputs[0].d[0];
    if (outputIndex == 0) *out = make_desc({batch, p_.max_voxels, p_.voxel_feature_num}, inputs[0].dtype);
    else if (outputIndex == 1) *out = make_desc({batch, p_.max_voxels, 4}, SESSD_DT_INT32);
    else if (outputIndex == 2) *out = make_desc({batch}, SESSD_DT_INT32);
    else return -1;
    return 0;
}

bool VoxelGeneratorPlugin::supportsFormatCombination(int pos, const TensorDesc* inOut, int, int) const {
    const TensorDesc& t = inOut[pos];
    switch (pos) {
        case 0: return t.dtype == SESSD_DT_FLOAT && t.format == 0;   // points
        case 1: return is_int32(t);                                   // points_size
        case 2: return is_feature_type(t);                            // voxels: fp32 as the reference, or fp16
        case 3: return is_int32(t);                                   // coors
        case 4: return is_int32(t);                                   // voxel_num
        default: return false;
    }
}

void VoxelGeneratorPlugin::configurePlugin(const TensorDesc* in, int nbInputs, const TensorDesc*, int) {
    if (in && nbInputs > 0) p_.point_feature_num = in[0].d[2];
    sessd_voxel_configure(&p_);   // grid = np_round((max - min) / voxel), voxelGenerator.cu:228-235
}

size_t VoxelGeneratorPlugin::getWorkspaceSize(const TensorDesc* inputs, int nbInputs, const TensorDesc*, int) const {
    if (!inputs || nbInputs < 1) return 0;
    return sessd_voxelize_workspace_bytes(&p_, inputs[0].d[0], inputs[0].d[1]);
}

int VoxelGeneratorPlugin::enqueue(const TensorDesc* inputDesc, const TensorDesc* outputDesc, const void* const* inputs,
                                  void* const* outputs, void* workspace, void* stream) {
    if (!inputDesc || !outputDesc) return SESSD_ERR_NULL;
    const int batch = inputDesc[0].d[0], max_points = inputDesc[0].d[1];
    return sessd_voxelize_enqueue(&p_, batch, max_points, feature_dtype(outputDesc[0]), inputs, outputs, workspace,
                                  sessd_voxelize_workspace_bytes(&p_, batch, max_points), stream);
}

int VoxelGeneratorPlugin::getOutputDataType(int index, const int32_t* inputTypes, int) const {
    return index == 0 ? inputTypes[0] : inputTypes[1];   // voxelGenerator.cu:544-550
}

void VoxelGeneratorPlugin::serialize(void* buffer) const { std::memcpy(buffer, &p_, sizeof(p_)); }

// ---------------------------------------------------------------- conv plugins

ConvPluginBase::ConvPluginBase(const sessd_conv_params& p, const float* weights, int weights_size) : p_(p) {
    dev_[0] = dev_[1] = nullptr;
    if (weights && weights_size > 0) weights_.assign(weights, weights + weights_size);
}

ConvPluginBase::~ConvPluginBase() { terminate(); }

void ConvPluginBase::terminate() {
    // the reference frees the same pointer twice (terminate + destructor, submConv3dlayer.cu:671-682)
    for (auto& d : dev_) {
        if (d) sessd_conv_weights_destroy(d);
        d = nullptr;
    }
}

int ConvPluginBase::ensureWeights(int dtype) {
    if (dev_[dtype]) return SESSD_OK;
    const size_t need = (size_t)p_.ksize[0] * p_.ksize[1] * p_.ksize[2] * p_.in_channel * p_.out_channel;
    if (weights_.size() < need) return SESSD_ERR_PARAM;
    // bare layer, as the reference plugin: BatchNorm and ReLU stay separate TensorRT layers
    return sessd_conv_weights_create(&p_, weights_.data(), nullptr, nullptr, 0, dtype, &dev_[dtype]);
}

bool ConvPluginBase::supportsFormatCombination(int pos, const TensorDesc* inOut, int nbInputs, int) const {
    const TensorDesc& t = inOut[pos];
    if (pos == 0) return is_feature_type(t);                     // features
    if (pos == 1 || pos == 2) return is_int32(t);                // coors, voxel_num
    if (pos == nbInputs) return is_feature_type(t) && t.dtype == inOut[0].dtype;  // output features
    return is_int32(t);                                          // output coors / voxel_num (strided layer)
}

size_t ConvPluginBase::getWorkspaceSize(const TensorDesc* inputs, int nbInputs, const TensorDesc*, int) const {
    if (!inputs || nbInputs < 1) return 0;
    return sessd_conv_workspace_bytes(&p_, inputs[0].d[0]);
}

int ConvPluginBase::enqueue(const TensorDesc* inputDesc, const TensorDesc*, const void* const* inputs,
                            void* const* outputs, void* workspace, void* stream) {
    if (!inputDesc) return SESSD_ERR_NULL;
    const int batch = inputDesc[0].d[0];
    const int dtype = feature_dtype(inputDesc[0]);
    int rc = ensureWeights(dtype);
    if (rc) return rc;
    const size_t bytes = sessd_conv_workspace_bytes(&p_, batch);
    return p_.subm ? sessd_subm_conv_enqueue(&p_, dev_[dtype], batch, inputs, outputs, workspace, bytes, stream)
                   : sessd_sparse_conv_enqueue(&p_, dev_[dtype], batch, inputs, outputs, workspace, bytes, stream);
}

int ConvPluginBase::getOutputDataType(int index, const int32_t* inputTypes, int) const {
    return index == 0 ? inputTypes[0] : inputTypes[1];
}

static sessd_conv_params subm_params(int in_channel, int out_channel, int max_voxels, int feature_num, int ox, int oy,
                                     int oz, int sx, int sy, int sz, int ksize, int padding, int dilation,
                                     int out_padding) {
    sessd_conv_params p{};
    p.in_channel = in_channel; p.out_channel = out_channel; p.max_voxels = max_voxels; p.feature_num = feature_num;
    p.out_shape_x = ox; p.out_shape_y = oy; p.out_shape_z = oz;
    p.spatial_shape_x = sx; p.spatial_shape_y = sy; p.spatial_shape_z = sz;
    for (int j = 0; j < 3; ++j) { p.ksize[j] = ksize; p.stride[j] = 1; p.padding[j] = padding; }
    p.dilation = dilation; p.out_padding = out_padding; p.subm = 1;
    return p;
}

SubmConv3dLayerPlugin::SubmConv3dLayerPlugin(int in_channel, int out_channel, int max_voxels, int feature_num,
                                             int out_shape_x, int out_shape_y, int out_shape_z, int spatial_shape_x,
                                             int spatial_shape_y, int spatial_shape_z, int ksize, int stride,
                                             int padding, int dilation, int out_padding, int weights_size,
                                             const float* weights)
    : ConvPluginBase(subm_params(in_channel, out_channel, max_voxels, feature_num, out_shape_x, out_shape_y,
                                 out_shape_z, spatial_shape_x, spatial_shape_y, spatial_shape_z, ksize, padding,
                                 dilation, out_padding),
                     weights, weights_size),
      stride_(stride) {}

static SubmConv3dLayerPlugin* subm_from_blob(const void* data, size_t length) {
    // 16 ints then the weights (submConv3dlayer.cu:154-186)
    if (!data || length < 16 * sizeof(int32_t)) return nullptr;
    const char* d = static_cast<const char*>(data);
    int v[16];
    for (int& x : v) x = get<int32_t>(d);
    if (v[15] < 0 || length < 16 * sizeof(int32_t) + (size_t)v[15] * sizeof(float)) return nullptr;
    std::vector<float> w((size_t)v[15]);
    if (v[15]) std::memcpy(w.data(), d, (size_t)v[15] * sizeof(float));
    return new SubmConv3dLayerPlugin(v[0], v[1], v[2], v[3], v[4], v[5], v[6], v[7], v[8], v[9], v[10], v[11], v[12],
                                     v[13], v[14], v[15], w.data());
}

SubmConv3dLayerPlugin::SubmConv3dLayerPlugin(const void* data, size_t length)
    : ConvPluginBase(sessd_conv_params{}, nullptr, 0), stride_(1) {
    if (SubmConv3dLayerPlugin* t = subm_from_blob(data, length)) {
        p_ = t->p_;
        weights_ = t->weights_;
        stride_ = t->stride_;
        delete t;
    }
}

PluginBase* SubmConv3dLayerPlugin::clone() const {
    return new SubmConv3dLayerPlugin(p_.in_channel, p_.out_channel, p_.max_voxels, p_.feature_num, p_.out_shape_x,
                                     p_.out_shape_y, p_.out_shape_z, p_.spatial_shape_x, p_.spatial_shape_y,
                                     p_.spatial_shape_z, p_.ksize[0], stride_, p_.padding[0], p_.dilation,
                                     p_.out_padding, (int)weights_.size(), weights_.data());
}

int SubmConv3dLayerPlugin::getOutputDimensions(int outputIndex, const TensorDesc* inputs, int nbInputs,
                                               TensorDesc* out) const {
    if (!inputs || nbInputs < 1 || !out || outputIndex != 0) return -1;
    *out = make_desc({inputs[0].d[0], p_.max_voxels, p_.out_channel}, inputs[0].dtype);
    return 0;
}

size_t SubmConv3dLayerPlugin::getSerializationSize() const {
    return weights_.size() * sizeof(float) + 16 * sizeof(int32_t);   // submConv3dlayer.cu:684-687
}

void SubmConv3dLayerPlugin::serialize(void* buffer) const {
    char* d = static_cast<char*>(buffer);
    const int32_t v[16] = {p_.in_channel, p_.out_channel, p_.max_voxels, p_.feature_num, p_.out_shape_x,
                           p_.out_shape_y, p_.out_shape_z, p_.spatial_shape_x, p_.spatial_shape_y, p_.spatial_shape_z,
                           p_.ksize[0], stride_, p_.padding[0], p_.dilation, p_.out_padding, (int32_t)weights_.size()};
    for (int32_t x : v) put<int32_t>(d, x);
    if (!weights_.empty()) std::memcpy(d, weights_.data(), weights_.size() * sizeof(float));
}

static sessd_conv_params sparse_params(int in_channel, int out_channel, int max_voxels, int feature_num, int ox, int oy,
                                       int oz, int sx, int sy, int sz, int k0, int k1, int k2, int s0, int s1, int s2,
                                       int p0, int p1, int p2, int dilation, int out_padding) {
    sessd_conv_params p{};
    p.in_channel = in_channel; p.out_channel = out_channel; p.max_voxels = max_voxels; p.feature_num = feature_num;
    p.out_shape_x = ox; p.out_shape_y = oy; p.out_shape_z = oz;
    p.spatial_shape_x = sx; p.spatial_shape_y = sy; p.spatial_shape_z = sz;
    p.ksize[0] = k0; p.ksize[1] = k1; p.ksize[2] = k2;
    p.stride[0] = s0; p.stride[1] = s1; p.stride[2] = s2;
    p.padding[0] = p0; p.padding[1] = p1; p.padding[2] = p2;
    p.dilation = dilation; p.out_padding = out_padding; p.subm = 0;
    return p;
}

SparseConv3dLayerPlugin::SparseConv3dLayerPlugin(int in_channel, int out_channel, int max_voxels, int feature_num,
                                                 int out_shape_x, int out_shape_y, int out_shape_z,
                                                 int spatial_shape_x, int spatial_shape_y, int spatial_shape_z,
                                                 int ksize0, int ksize1, int ksize2, int stride0, int stride1,
                                                 int stride2, int padding0, int padding1, int padding2, int dilation,
                                                 int out_padding, int weights_size, const float* weights)
    : ConvPluginBase(sparse_params(in_channel, out_channel, max_voxels, feature_num, out_shape_x, out_shape_y,
                                   out_shape_z, spatial_shape_x, spatial_shape_y, spatial_shape_z, ksize0, ksize1,
                                   ksize2, stride0, stride1, stride2, padding0, padding1, padding2, dilation,
                                   out_padding),
                     weights, weights_size) {}

SparseConv3dLayerPlugin::SparseConv3dLayerPlugin(const void* data, size_t length)
    : ConvPluginBase(sessd_conv_params{}, nullptr, 0) {
    // 22 ints then the weights (sparseConv3dlayer.cu:165-200)
    if (!data || length < 22 * sizeof(int32_t)) return;
    const char* d = static_cast<const char*>(data);
    int v[22];
    for (int& x : v) x = get<int32_t>(d);
    if (v[21] < 0 || length < 22 * sizeof(int32_t) + (size_t)v[21] * sizeof(float)) return;
    p_ = sparse_params(v[0], v[1], v[2], v[3], v[4], v[5], v[6], v[7], v[8], v[9], v[10], v[11], v[12], v[13], v[14],
                       v[15], v[16], v[17], v[18], v[19], v[20]);
    weights_.resize((size_t)v[21]);
    if (v[21]) std::memcpy(weights_.data(), d, (size_t)v[21] * sizeof(float));
}

PluginBase* SparseConv3dLayerPlugin::clone() const {
    return new SparseConv3dLayerPlugin(p_.in_channel, p_.out_channel, p_.max_voxels, p_.feature_num, p_.out_shape_x,
                                       p_.out_shape_y, p_.out_shape_z, p_.spatial_shape_x, p_.spatial_shape_y,
                                       p_.spatial_shape_z, p_.ksize[0], p_.ksize[1], p_.ksize[2], p_.stride[0],
                                       p_.stride[1], p_.stride[2], p_.padding[0], p_.padding[1], p_.padding[2],
                                       p_.dilation, p_.out_padding, (int)weights_.size(), weights_.data());
}

int SparseConv3dLayerPlugin::getOutputDimensions(int outputIndex, const TensorDesc* inputs, int nbInputs,
                                                 TensorDesc* out) const {
    if (!inputs || nbInputs < 1 || !out) return -1;
    const int batch = inputs[0].d[0];
    if (outputIndex == 0) *out = make_desc({batch, p_.max_voxels, p_.out_channel}, inputs[0].dtype);
    else if (outputIndex == 1) *out = make_desc({batch, p_.max_voxels, 4}, SESSD_DT_INT32);
    else if (outputIndex == 2) *out = make_desc({batch}, SESSD_DT_INT32);
    else return -1;
    return 0;
}

size_t SparseConv3dLayerPlugin::getSerializationSize() const {
    return weights_.size() * sizeof(float) + 22 * sizeof(int32_t);   // sparseConv3dlayer.cu:863-866
}

void SparseConv3dLayerPlugin::serialize(void* buffer) const {
    char* d = static_cast<char*>(buffer);
    const int32_t v[22] = {p_.in_channel, p_.out_channel, p_.max_voxels, p_.feature_num, p_.out_shape_x,
                           p_.out_shape_y, p_.out_shape_z, p_.spatial_shape_x, p_.spatial_shape_y, p_.spatial_shape_z,
                           p_.ksize[0], p_.ksize[1], p_.ksize[2], p_.stride[0], p_.stride[1], p_.stride[2],
                           p_.padding[0], p_.padding[1], p_.padding[2], p_.dilation, p_.out_padding,
                           (int32_t)weights_.size()};
    for (int32_t x : v) put<int32_t>(d, x);
    if (!weights_.empty()) std::memcpy(d, weights_.data(), weights_.size() * sizeof(float));
}

// ---------------------------------------------------------------- Sparse2DensePlugin

Sparse2DensePlugin::Sparse2DensePlugin(int x, int y, int z, int channel) { p_ = sessd_s2d_params{x, y, z, channel}; }

Sparse2DensePlugin::Sparse2DensePlugin(const void* data, size_t length) {
    std::memset(&p_, 0, sizeof(p_));
    if (data && length >= sizeof(p_)) std::memcpy(&p_, data, sizeof(p_));
}

PluginBase* Sparse2DensePlugin::clone() const { return new Sparse2DensePlugin(*this); }

int Sparse2DensePlugin::getOutputDimensions(int outputIndex, const TensorDesc* inputs, int nbInputs,
                                            TensorDesc* out) const {
    if (!inputs || nbInputs < 1 || !out || outputIndex != 0) return -1;
    // [B, C*D, H, W] (sparse2Dense.cu:127-143)
    *out = make_desc({inputs[0].d[0], p_.feature_map_size_z * p_.feature_map_channel, p_.feature_map_size_y,
                      p_.feature_map_size_x},
                     inputs[0].dtype);
    return 0;
}

bool Sparse2DensePlugin::supportsFormatCombination(int pos, const TensorDesc* inOut, int, int) const {
    const TensorDesc& t = inOut[pos];
    if (pos == 0) return is_feature_type(t);
    if (pos == 1 || pos == 2) return is_int32(t);
    if (pos == 3) return is_feature_type(t) && t.dtype == inOut[0].dtype;
    return false;
}

int Sparse2DensePlugin::enqueue(const TensorDesc* inputDesc, const TensorDesc*, const void* const* inputs,
                                void* const* outputs, void*, void* stream) {
    if (!inputDesc) return SESSD_ERR_NULL;
    return sessd_sparse2dense_enqueue(&p_, inputDesc[0].d[0], inputDesc[0].d[1], feature_dtype(inputDesc[0]), inputs,
                                      outputs, nullptr, 0, stream);
}

int Sparse2DensePlugin::getOutputDataType(int, const int32_t* inputTypes, int) const { return inputTypes[0]; }

void Sparse2DensePlugin::serialize(void* buffer) const { std::memcpy(buffer, &p_, sizeof(p_)); }

// ---------------------------------------------------------------- ZeroPad2dPlugin

ZeroPad2dPlugin::ZeroPad2dPlugin(int top, int bottom, int left, int right) { p_ = sessd_pad2d_params{top, bottom, left, right}; }

ZeroPad2dPlugin::ZeroPad2dPlugin(const void* data, size_t length) {
    std::memset(&p_, 0, sizeof(p_));
    if (data && length >= sizeof(p_)) std::memcpy(&p_, data, sizeof(p_));   // zeroPad2d.cu:111-118
}

PluginBase* ZeroPad2dPlugin::clone() const { return new ZeroPad2dPlugin(*this); }

int ZeroPad2dPlugin::getOutputDimensions(int outputIndex, const TensorDesc* inputs, int nbInputs, TensorDesc* out) const {
    if (!inputs || nbInputs < 1 || !out || outputIndex != 0) return -1;
    *out = make_desc({inputs[0].d[0], inputs[0].d[1], inputs[0].d[2] + p_.top + p_.bottom,
                      inputs[0].d[3] + p_.left + p_.right},
                     inputs[0].dtype);   // zeroPad2d.cu:127-151
    return 0;
}

bool ZeroPad2dPlugin::supportsFormatCombination(int pos, const TensorDesc* inOut, int, int) const {
    if (pos == 0) return is_feature_type(inOut[0]);
    if (pos == 1) return is_feature_type(inOut[1]) && inOut[1].dtype == inOut[0].dtype;
    return false;
}

int ZeroPad2dPlugin::enqueue(const TensorDesc* inputDesc, const TensorDesc*, const void* const* inputs,
                             void* const* outputs, void*, void* stream) {
    if (!inputDesc) return SESSD_ERR_NULL;
    return sessd_zero_pad2d_enqueue(&p_, inputDesc[0].d[0], inputDesc[0].d[1], inputDesc[0].d[2], inputDesc[0].d[3],
                                    feature_dtype(inputDesc[0]), inputs, outputs, stream);
}

int ZeroPad2dPlugin::getOutputDataType(int, const int32_t* inputTypes, int) const { return inputTypes[0]; }

void ZeroPad2dPlugin::serialize(void* buffer) const { std::memcpy(buffer, &p_, sizeof(p_)); }

// ---------------------------------------------------------------- GenerateAnchorDecodePlugin

GenerateAnchorDecodePlugin::GenerateAnchorDecodePlugin(float min_x_range, float max_x_range, float min_y_range,
                                                       float max_y_range, float min_z_range, float max_z_range,
                                                       int feature_map_height, int feature_map_width, float car_length,
                                                       float car_width, float car_height, float direction_angle_0,
                                                       float direction_angle_1, int direction_angle_num) {
    // argument order of the reference constructor (generateAnchorDecode.cu:105-114)
    p_ = sessd_anchor_params{min_x_range, max_x_range, min_y_range, max_y_range, min_z_range, max_z_range,
                             feature_map_height, feature_map_width, car_length, car_width, car_height,
                             direction_angle_0, direction_angle_1, direction_angle_num};
}

GenerateAnchorDecodePlugin::GenerateAnchorDecodePlugin(const void* data, size_t length) {
    std::memset(&p_, 0, sizeof(p_));
    if (data && length >= sizeof(p_)) std::memcpy(&p_, data, sizeof(p_));   // generateAnchorDecode.cu:116-137
}

PluginBase* GenerateAnchorDecodePlugin::clone() const { return new GenerateAnchorDecodePlugin(*this); }

int GenerateAnchorDecodePlugin::getOutputDimensions(int outputIndex, const TensorDesc* inputs, int nbInputs,
                                                    TensorDesc* out) const {
    if (!inputs || nbInputs < 1 || !out || outputIndex != 0) return -1;
    *out = make_desc({inputs[0].d[0], inputs[0].d[1], inputs[0].d[2]}, inputs[0].dtype);   // :150-171
    return 0;
}

bool GenerateAnchorDecodePlugin::supportsFormatCombination(int pos, const TensorDesc* inOut, int, int) const {
    return (pos == 0 || pos == 1) && inOut[pos].dtype == SESSD_DT_FLOAT && inOut[pos].format == 0;   // :173-187
}

int GenerateAnchorDecodePlugin::enqueue(const TensorDesc* inputDesc, const TensorDesc*, const void* const* inputs,
                                        void* const* outputs, void*, void* stream) {
    if (!inputDesc) return SESSD_ERR_NULL;
    return sessd_anchor_decode_enqueue(&p_, inputDesc[0].d[0], inputs, outputs, stream);
}

int GenerateAnchorDecodePlugin::getOutputDataType(int, const int32_t* inputTypes, int) const { return inputTypes[0]; }

void GenerateAnchorDecodePlugin::serialize(void* buffer) const {
    // The reference writes max_y_range_ where max_z_range_ belongs (generateAnchorDecode.cu:409), so a
    // deserialised plugin has max_z = max_y; the blob is reproduced byte for byte (max_z is never used).
    sessd_anchor_params blob = p_;
    blob.max_z = p_.max_y;
    std::memcpy(buffer, &blob, sizeof(blob));
}

// ---------------------------------------------------------------- FilterBoxByScorePlugin

FilterBoxByScorePlugin::FilterBoxByScorePlugin(int feature_map_height, int feature_map_width, int direction_angle_num,
                                               int max_box_num, float score_threshold, float direction_offset) {
    p_ = sessd_filter_params{feature_map_height, feature_map_width, direction_angle_num, max_box_num, score_threshold,
                             direction_offset};
}

FilterBoxByScorePlugin::FilterBoxByScorePlugin(const void* data, size_t length) {
    std::memset(&p_, 0, sizeof(p_));
    if (data && length >= sizeof(p_)) std::memcpy(&p_, data, sizeof(p_));   // filterBoxByScore.cu:115-128
}

PluginBase* FilterBoxByScorePlugin::clone() const { return new FilterBoxByScorePlugin(*this); }

int FilterBoxByScorePlugin::getOutputDimensions(int outputIndex, const TensorDesc* inputs, int nbInputs,
                                                TensorDesc* out) const {
    if (!inputs || nbInputs < 4 || !out) return -1;
    const int batch = inputs[0].d[0];
    switch (outputIndex) {   // filterBoxByScore.cu:138-199
        case 0: *out = make_desc({batch, p_.max_box_num, inputs[0].d[2] + 2}, inputs[0].dtype); return 0;
        case 1: *out = make_desc({batch, p_.max_box_num}, inputs[0].dtype); return 0;
        case 2: *out = make_desc({batch, p_.max_box_num, inputs[2].d[2]}, inputs[0].dtype); return 0;
        case 3: *out = make_desc({batch, p_.max_box_num, 1}, inputs[0].dtype); return 0;
        case 4: *out = make_desc({batch, 1}, SESSD_DT_INT32); return 0;
        default: return -1;
    }
}

bool FilterBoxByScorePlugin::supportsFormatCombination(int pos, const TensorDesc* inOut, int, int) const {
    if (pos < 0 || pos > 8) return false;
    const TensorDesc& t = inOut[pos];
    return t.format == 0 && t.dtype == (pos == 8 ? SESSD_DT_INT32 : SESSD_DT_FLOAT);   // :202-243
}

size_t FilterBoxByScorePlugin::getWorkspaceSize(const TensorDesc* inputs, int nbInputs, const TensorDesc*, int) const {
    if (!inputs || nbInputs < 1) return 0;
    return sessd_filter_boxes_workspace_bytes(&p_, inputs[0].d[0]);
}

int FilterBoxByScorePlugin::enqueue(const TensorDesc* inputDesc, const TensorDesc*, const void* const* inputs,
                                    void* const* outputs, void* workspace, void* stream) {
    if (!inputDesc) return SESSD_ERR_NULL;
    const int batch = inputDesc[0].d[0];
    return sessd_filter_boxes_enqueue(&p_, batch, inputs, outputs, workspace,
                                      sessd_filter_boxes_workspace_bytes(&p_, batch), stream);
}

int FilterBoxByScorePlugin::getOutputDataType(int index, const int32_t* inputTypes, int) const {
    return index == 4 ? SESSD_DT_INT32 : inputTypes[0];   // filterBoxByScore.cu:384-390
}

void FilterBoxByScorePlugin::serialize(void* buffer) const { std::memcpy(buffer, &p_, sizeof(p_)); }

// ---------------------------------------------------------------- creators

namespace {

const Field* find_field(const Field* fields, int n, const char* name) {
    for (int i = 0; i < n; ++i)
        if (fields[i].name && !std::strcmp(fields[i].name, name)) return &fields[i];
    return nullptr;
}
int int_at(const Field* f, int i, int dflt = 0) { return (f && f->data) ? static_cast<const int32_t*>(f->data)[i] : dflt; }
float float_at(const Field* f, int i) { return (f && f->data) ? static_cast<const float*>(f->data)[i] : 0.f; }

class VoxelCreator : public PluginCreator {
public:
    const char* getPluginName() const override { return "VoxelGeneratorPlugin"; }
    const std::vector<std::string>& getFieldNames() const override {
        static const std::vector<std::string> n = {"max_num_points_per_voxel", "max_voxels", "point_cloud_range",
                                                   "voxel_feature_num", "voxel_size"};   // voxelGenerator.cu:624-628
        return n;
    }
    PluginBase* createPlugin(const char*, const Field* f, int n) const override {
        const Field *pts = find_field(f, n, "max_num_points_per_voxel"), *mv = find_field(f, n, "max_voxels"),
                    *rng = find_field(f, n, "point_cloud_range"), *vf = find_field(f, n, "voxel_feature_num"),
                    *vs = find_field(f, n, "voxel_size");
        if (!pts || !mv || !rng || !vf || !vs) return nullptr;
        // range arrives as (xmin, ymin, zmin, xmax, ymax, zmax) and is re-ordered exactly as
        // voxelGenerator.cu:697-699 does
        return new VoxelGeneratorPlugin(int_at(mv, 0), int_at(pts, 0), int_at(vf, 0), float_at(rng, 0), float_at(rng, 3),
                                        float_at(rng, 1), float_at(rng, 4), float_at(rng, 2), float_at(rng, 5),
                                        float_at(vs, 0), float_at(vs, 1), float_at(vs, 2));
    }
    PluginBase* deserializePlugin(const char*, const void* d, size_t len) const override {
        return len >= sizeof(sessd_voxel_params) ? new VoxelGeneratorPlugin(d, len) : nullptr;
    }
};

const std::vector<std::string>& conv_field_names() {
    static const std::vector<std::string> n = {"in_channel", "out_channel", "max_voxels", "feature_num", "out_shape",
                                               "spatial_shape", "ksize", "stride", "padding", "dilation",
                                               "out_padding", "weights"};   // submConv3dlayer.cu:737-748
    return n;
}

class SubmCreator : public PluginCreator {
public:
    const char* getPluginName() const override { return "SubmConv3dLayerPlugin"; }
    const std::vector<std::string>& getFieldNames() const override { return conv_field_names(); }
    PluginBase* createPlugin(const char*, const Field* f, int n) const override {
        auto F = [&](const char* name) { return find_field(f, n, name); };
        const Field* w = F("weights");
        if (!F("in_channel") || !F("out_channel") || !F("max_voxels") || !F("out_shape") || !F("ksize") || !w || !w->data)
            return nullptr;
        const int in = int_at(F("in_channel"), 0), out = int_at(F("out_channel"), 0), k = int_at(F("ksize"), 0);
        const Field *os = F("out_shape"), *ss = F("spatial_shape") ? F("spatial_shape") : os;
        const int wsize = in * out * k * k * k;   // submConv3dlayer.cu:873
        // shapes arrive in (x, y, z) order (submConv3dlayer.cu:827-840)
        return new SubmConv3dLayerPlugin(in, out, int_at(F("max_voxels"), 0), int_at(F("feature_num"), 0, in),
                                         int_at(os, 0), int_at(os, 1), int_at(os, 2), int_at(ss, 0), int_at(ss, 1),
                                         int_at(ss, 2), k, int_at(F("stride"), 0, 1), int_at(F("padding"), 0, 0),
                                         int_at(F("dilation"), 0, 1), int_at(F("out_padding"), 0, 0), wsize,
                                         static_cast<const float*>(w->data));
    }
    PluginBase* deserializePlugin(const char*, const void* d, size_t len) const override {
        return subm_from_blob(d, len);
    }
};

class SparseCreator : public PluginCreator {
public:
    const char* getPluginName() const override { return "SparseConv3dLayerPlugin"; }
    const std::vector<std::string>& getFieldNames() const override { return conv_field_names(); }
    PluginBase* createPlugin(const char*, const Field* f, int n) const override {
        auto F = [&](const char* name) { return find_field(f, n, name); };
        const Field* w = F("weights");
        if (!F("in_channel") || !F("out_channel") || !F("max_voxels") || !F("out_shape") || !F("spatial_shape") ||
            !F("ksize") || !F("stride") || !F("padding") || !w || !w->data)
            return nullptr;
        const int in = int_at(F("in_channel"), 0), out = int_at(F("out_channel"), 0);
        const Field *os = F("out_shape"), *ss = F("spatial_shape"), *k = F("ksize"), *s = F("stride"), *p = F("padding");
        const int wsize = in * out * int_at(k, 0) * int_at(k, 1) * int_at(k, 2);
        // ksize/stride/padding arrive as (z, y, x) triples = ksize0..2 (sparseConv3dlayer.cu:1028-1048)
        return new SparseConv3dLayerPlugin(in, out, int_at(F("max_voxels"), 0), int_at(F("feature_num"), 0, in),
                                           int_at(os, 0), int_at(os, 1), int_at(os, 2), int_at(ss, 0), int_at(ss, 1),
                                           int_at(ss, 2), int_at(k, 0), int_at(k, 1), int_at(k, 2), int_at(s, 0),
                                           int_at(s, 1), int_at(s, 2), int_at(p, 0), int_at(p, 1), int_at(p, 2),
                                           int_at(F("dilation"), 0, 1), int_at(F("out_padding"), 0, 0), wsize,
                                           static_cast<const float*>(w->data));
    }
    PluginBase* deserializePlugin(const char*, const void* d, size_t len) const override {
        if (!d || len < 22 * sizeof(int32_t)) return nullptr;
        return new SparseConv3dLayerPlugin(d, len);
    }
};

class S2DCreator : public PluginCreator {
public:
    const char* getPluginName() const override { return "Sparse2DensePlugin"; }
    const std::vector<std::string>& getFieldNames() const override {
        static const std::vector<std::string> n = {"feature_map_size", "feature_map_channel"};   // sparse2Dense.cu:321-365
        return n;
    }
    PluginBase* createPlugin(const char*, const Field* f, int n) const override {
        const Field *sz = find_field(f, n, "feature_map_size"), *ch = find_field(f, n, "feature_map_channel");
        if (!sz || !ch) return nullptr;
        return new Sparse2DensePlugin(int_at(sz, 0), int_at(sz, 1), int_at(sz, 2), int_at(ch, 0));   // (x, y, z)
    }
    PluginBase* deserializePlugin(const char*, const void* d, size_t len) const override {
        return len >= sizeof(sessd_s2d_params) ? new Sparse2DensePlugin(d, len) : nullptr;
    }
};

class PadCreator : public PluginCreator {
public:
    const char* getPluginName() const override { return "ZeroPad2dPlugin"; }
    const std::vector<std::string>& getFieldNames() const override {
        static const std::vector<std::string> n = {"zero_padding_2d_size"};   // zeroPad2d.cu:315
        return n;
    }
    PluginBase* createPlugin(const char*, const Field* f, int n) const override {
        const Field* sz = find_field(f, n, "zero_padding_2d_size");
        // a missing field leaves all four at zero in the reference (zeroPad2d.cu:341-356)
        return new ZeroPad2dPlugin(int_at(sz, 0), int_at(sz, 1), int_at(sz, 2), int_at(sz, 3));   // top, bottom, left, right
    }
    PluginBase* deserializePlugin(const char*, const void* d, size_t len) const override {
        return len >= sizeof(sessd_pad2d_params) ? new ZeroPad2dPlugin(d, len) : nullptr;
    }
};

class AnchorCreator : public PluginCreator {
public:
    const char* getPluginName() const override { return "GenerateAnchorDecodePlugin"; }
    const std::vector<std::string>& getFieldNames() const override {
        static const std::vector<std::string> n = {"point_cloud_range", "feature_map_size", "car_size", "direction_angle",
                                                   "direction_angle_num"};   // generateAnchorDecode.cu:443-447
        return n;
    }
    PluginBase* createPlugin(const char*, const Field* f, int n) const override {
        const Field *rng = find_field(f, n, "point_cloud_range"), *sz = find_field(f, n, "feature_map_size"),
                    *car = find_field(f, n, "car_size"), *ang = find_field(f, n, "direction_angle"),
                    *num = find_field(f, n, "direction_angle_num");
        if (!rng || !sz || !car || !ang || !num) return nullptr;
        // range arrives as (xmin, ymin, zmin, xmax, ymax, zmax), size as (height, width), car as
        // (length, width, height) (generateAnchorDecode.cu:492-527)
        return new GenerateAnchorDecodePlugin(float_at(rng, 0), float_at(rng, 3), float_at(rng, 1), float_at(rng, 4),
                                              float_at(rng, 2), float_at(rng, 5), int_at(sz, 0), int_at(sz, 1),
                                              float_at(car, 0), float_at(car, 1), float_at(car, 2), float_at(ang, 0),
                                              float_at(ang, 1), int_at(num, 0));
    }
    PluginBase* deserializePlugin(const char*, const void* d, size_t len) const override {
        return len >= sizeof(sessd_anchor_params) ? new GenerateAnchorDecodePlugin(d, len) : nullptr;
    }
};

class FilterCreator : public PluginCreator {
public:
    const char* getPluginName() const override { return "FilterBoxByScorePlugin"; }
    const std::vector<std::string>& getFieldNames() const override {
        static const std::vector<std::string> n = {"feature_map_size", "direction_angle_num", "max_box_num",
                                                   "score_threshold", "direction_offset"};   // filterBoxByScore.cu:466-470
        return n;
    }
    PluginBase* createPlugin(const char*, const Field* f, int n) const override {
        const Field *sz = find_field(f, n, "feature_map_size"), *num = find_field(f, n, "direction_angle_num"),
                    *mb = find_field(f, n, "max_box_num"), *thr = find_field(f, n, "score_threshold"),
                    *off = find_field(f, n, "direction_offset");
        if (!sz || !num || !mb || !thr) return nullptr;
        return new FilterBoxByScorePlugin(int_at(sz, 0), int_at(sz, 1), int_at(num, 0), int_at(mb, 0), float_at(thr, 0),
                                          float_at(off, 0));
    }
    PluginBase* deserializePlugin(const char*, const void* d, size_t len) const override {
        return len >= sizeof(sessd_filter_params) ? new FilterBoxByScorePlugin(d, len) : nullptr;
    }
};

}  // namespace

const PluginCreator* getPluginCreator(const char* name, const char* version) {
    static const VoxelCreator voxel;
    static const SubmCreator subm;
    static const SparseCreator sparse;
    static const S2DCreator s2d;
    static const PadCreator pad;
    static const AnchorCreator anchor;
    static const FilterCreator filter;
    static const PluginCreator* all[] = {&voxel, &subm, &sparse, &s2d, &pad, &anchor, &filter};
    if (!name || (version && std::strcmp(version, "1"))) return nullptr;
    for (const PluginCreator* c : all)
        if (!std::strcmp(c->getPluginName(), name)) return c;
    return nullptr;
}

}  // namespace plugin
}  // namespace sessd

// ---------------------------------------------------------------- C view

using sessd::plugin::PluginBase;
struct sessd_plugin {
    PluginBase* impl;
};

extern "C" {

int sessd_plugin_field_names(const char* plugin_name, char* buf, size_t cap) {
    const auto* c = sessd::plugin::getPluginCreator(plugin_name, "1");
    if (!c) return -1;
    std::string joined;
    for (const auto& n : c->getFieldNames()) joined += n + "\n";
    if (buf && cap) {
        std::strncpy(buf, joined.c_str(), cap - 1);
        buf[cap - 1] = 0;
    }
    return (int)c->getFieldNames().size();
}

sessd_plugin* sessd_plugin_create(const char* plugin_name, const char* layer_name, const sessd_plugin_field* fields,
                                  int nb_fields) {
    const auto* c = sessd::plugin::getPluginCreator(plugin_name, "1");
    if (!c || !fields || nb_fields < 0) return nullptr;
    PluginBase* p = c->createPlugin(layer_name, fields, nb_fields);
    return p ? new sessd_plugin{p} : nullptr;
}

sessd_plugin* sessd_plugin_deserialize(const char* plugin_name, const void* data, size_t length) {
    const auto* c = sessd::plugin::getPluginCreator(plugin_name, "1");
    if (!c || !data) return nullptr;
    PluginBase* p = c->deserializePlugin(plugin_name, data, length);
    return p ? new sessd_plugin{p} : nullptr;
}

sessd_plugin* sessd_plugin_clone(const sessd_plugin* p) {
    if (!p) return nullptr;
    PluginBase* c = p->impl->clone();
    return c ? new sessd_plugin{c} : nullptr;
}

void sessd_plugin_destroy(sessd_plugin* p) {
    if (!p) return;
    p->impl->destroy();
    delete p;
}

const char* sessd_plugin_type(const sessd_plugin* p) { return p ? p->impl->getPluginType() : nullptr; }
const char* sessd_plugin_version(const sessd_plugin* p) { return p ? p->impl->getPluginVersion() : nullptr; }
int sessd_plugin_nb_outputs(const sessd_plugin* p) { return p ? p->impl->getNbOutputs() : -1; }

int sessd_plugin_output_dims(const sessd_plugin* p, int output_index, const sessd_tensor_desc* inputs, int nb_inputs,
                             sessd_tensor_desc* out) {
    return p ? p->impl->getOutputDimensions(output_index, inputs, nb_inputs, out) : -1;
}

int sessd_plugin_output_dtype(const sessd_plugin* p, int output_index, const int32_t* input_types, int nb_inputs) {
    return (p && input_types) ? p->impl->getOutputDataType(output_index, input_types, nb_inputs) : -1;
}

int sessd_plugin_supports_format(const sessd_plugin* p, int pos, const sessd_tensor_desc* in_out, int nb_inputs,
                                 int nb_outputs) {
    if (!p || !in_out || pos < 0 || pos >= nb_inputs + nb_outputs) return 0;
    return p->impl->supportsFormatCombination(pos, in_out, nb_inputs, nb_outputs) ? 1 : 0;
}

void sessd_plugin_configure(sessd_plugin* p, const sessd_tensor_desc* in, int nb_inputs, const sessd_tensor_desc* out,
                            int nb_outputs) {
    if (p) p->impl->configurePlugin(in, nb_inputs, out, nb_outputs);
}

size_t sessd_plugin_workspace_size(const sessd_plugin* p, const sessd_tensor_desc* inputs, int nb_inputs,
                                   const sessd_tensor_desc* outputs, int nb_outputs) {
    return p ? p->impl->getWorkspaceSize(inputs, nb_inputs, outputs, nb_outputs) : 0;
}

int sessd_plugin_enqueue(sessd_plugin* p, const sessd_tensor_desc* input_desc, const sessd_tensor_desc* output_desc,
                         const void* const* inputs, void* const* outputs, void* workspace, void* stream) {
    if (!p) return SESSD_ERR_NULL;
    return p->impl->enqueue(input_desc, output_desc, inputs, outputs, workspace, stream);
}

size_t sessd_plugin_serialization_size(const sessd_plugin* p) { return p ? p->impl->getSerializationSize() : 0; }
void sessd_plugin_serialize(const sessd_plugin* p, void* buffer) {
    if (p && buffer) p->impl->serialize(buffer);
}

}  // extern "C"
