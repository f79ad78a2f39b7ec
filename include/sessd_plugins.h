/*
 * sessd_plugins.h - C view of the plugin layer that sits on top of sessd.h.
 *
 * The reference exposes the sparse front end as four TensorRT plugins (IPluginV2DynamicExt +
 * IPluginCreator): VoxelGeneratorPlugin (voxelGenerator.h:19-110), SubmConv3dLayerPlugin
 * (submConv3dlayer.h:19-121), SparseConv3dLayerPlugin (sparseConv3dlayer.h:18-126) and
 * Sparse2DensePlugin (sparse2Dense.h:18-86). se-ssd-ai-trt_b200/csrc/plugins.h holds C++ classes with
 * the same names, creator field names, method names, tensor orders, error behaviour (0 = ok from
 * enqueue) and byte-identical serialisation; they call the kernels only through sessd.h. TensorRT itself
 * is not needed to use them. The functions below drive those classes from C (and from the tests).
 */
#ifndef SESSD_PLUGINS_H_
#define SESSD_PLUGINS_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Data types / field types use TensorRT's numeric values (DataType, PluginFieldType). */
enum { SESSD_DT_FLOAT = 0, SESSD_DT_HALF = 1, SESSD_DT_INT32 = 3 };
enum { SESSD_PF_FLOAT32 = 1, SESSD_PF_INT32 = 4 };

/* Stand-in for nvinfer1::PluginTensorDesc: dims, data type, format (0 = linear). */
typedef struct sessd_tensor_desc {
    int32_t nb_dims;
    int32_t d[8];
    int32_t dtype;
    int32_t format;
} sessd_tensor_desc;

/* Stand-in for nvinfer1::PluginField. As in the reference, `length` is not trusted: arrays are read by
 * pointer with their documented length (e.g. out_shape = 3 ints in x, y, z order). */
typedef struct sessd_plugin_field {
    const char* name;
    const void* data;
    int32_t type;
    int32_t length;
} sessd_plugin_field;

typedef struct sessd_plugin sessd_plugin;

/* IPluginCreator::getFieldNames of the creator registered under `plugin_name` ("VoxelGeneratorPlugin",
 * "SubmConv3dLayerPlugin", "SparseConv3dLayerPlugin", "Sparse2DensePlugin"; version "1"): newline separated
 * names written to buf; returns the number of fields or -1 for an unknown plugin. */
int sessd_plugin_field_names(const char* plugin_name, char* buf, size_t cap);
/* IPluginCreator::createPlugin / deserializePlugin. Null on failure. */
sessd_plugin* sessd_plugin_create(const char* plugin_name, const char* layer_name, const sessd_plugin_field* fields,
                                  int nb_fields);
sessd_plugin* sessd_plugin_deserialize(const char* plugin_name, const void* data, size_t length);
/* IPluginV2DynamicExt members. */
sessd_plugin* sessd_plugin_clone(const sessd_plugin* p);
void sessd_plugin_destroy(sessd_plugin* p);
const char* sessd_plugin_type(const sessd_plugin* p);
const char* sessd_plugin_version(const sessd_plugin* p);
int sessd_plugin_nb_outputs(const sessd_plugin* p);
int sessd_plugin_output_dims(const sessd_plugin* p, int output_index, const sessd_tensor_desc* inputs, int nb_inputs,
                             sessd_tensor_desc* out);
int sessd_plugin_output_dtype(const sessd_plugin* p, int output_index, const int32_t* input_types, int nb_inputs);
int sessd_plugin_supports_format(const sessd_plugin* p, int pos, const sessd_tensor_desc* in_out, int nb_inputs,
                                 int nb_outputs);
void sessd_plugin_configure(sessd_plugin* p, const sessd_tensor_desc* in, int nb_inputs, const sessd_tensor_desc* out,
                            int nb_outputs);
size_t sessd_plugin_workspace_size(const sessd_plugin* p, const sessd_tensor_desc* inputs, int nb_inputs,
                                   const sessd_tensor_desc* outputs, int nb_outputs);
int sessd_plugin_enqueue(sessd_plugin* p, const sessd_tensor_desc* input_desc, const sessd_tensor_desc* output_desc,
                         const void* const* inputs, void* const* outputs, void* workspace, void* stream);
size_t sessd_plugin_serialization_size(const sessd_plugin* p);
void sessd_plugin_serialize(const sessd_plugin* p, void* buffer);

/* 1 when the library was built with TensorRT's headers present, i.e. when it also holds the seven
 * nvinfer1::IPluginV2DynamicExt classes over the plugins above and registers their creators with
 * REGISTER_TENSORRT_PLUGIN as the reference does (voxelGenerator.h:111 and the sibling headers); 0 otherwise. */
int sessd_tensorrt_shim_present(void);

#ifdef __cplusplus
}
#endif
#endif /* SESSD_PLUGINS_H_ */
