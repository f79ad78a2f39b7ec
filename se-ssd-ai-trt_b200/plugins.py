"""ctypes view of the plugin layer (include/sessd_plugins.h): the reference's four TensorRT plugins,
re-hosted on the C ABI. Used by the tests; a TensorRT shim would call the same C++ classes directly."""
from __future__ import annotations

import ctypes as C

import numpy as np

DT_FLOAT, DT_HALF, DT_INT32 = 0, 1, 3
PF_FLOAT32, PF_INT32 = 1, 4

PLUGIN_EXPORTS = (
    "sessd_plugin_field_names", "sessd_plugin_create", "sessd_plugin_deserialize", "sessd_plugin_clone",
    "sessd_plugin_destroy", "sessd_plugin_type", "sessd_plugin_version", "sessd_plugin_nb_outputs",
    "sessd_plugin_output_dims", "sessd_plugin_output_dtype", "sessd_plugin_supports_format",
    "sessd_plugin_configure", "sessd_plugin_workspace_size", "sessd_plugin_enqueue",
    "sessd_plugin_serialization_size", "sessd_plugin_serialize",
)


class TensorDesc(C.Structure):
    _fields_ = [("nb_dims", C.c_int32), ("d", C.c_int32 * 8), ("dtype", C.c_int32), ("format", C.c_int32)]

    @classmethod
    def of(cls, dims, dtype, fmt=0):
        t = cls()
        t.nb_dims, t.dtype, t.format = len(dims), dtype, fmt
        for i, v in enumerate(dims):
            t.d[i] = v
        return t

    def dims(self):
        return tuple(self.d[i] for i in range(self.nb_dims))


class PluginField(C.Structure):
    _fields_ = [("name", C.c_char_p), ("data", C.c_void_p), ("type", C.c_int32), ("length", C.c_int32)]


def _lib():
    from . import lib

    L = lib()
    if not getattr(L, "_plugins_bound", False):
        for n in ("sessd_plugin_create", "sessd_plugin_deserialize", "sessd_plugin_clone"):
            getattr(L, n).restype = C.c_void_p
        for n in ("sessd_plugin_type", "sessd_plugin_version"):
            getattr(L, n).restype = C.c_char_p
        for n in ("sessd_plugin_workspace_size", "sessd_plugin_serialization_size"):
            getattr(L, n).restype = C.c_size_t
        L._plugins_bound = True
    return L


def field_names(plugin_name: str):
    buf = C.create_string_buffer(1024)
    n = _lib().sessd_plugin_field_names(plugin_name.encode(), buf, C.c_size_t(len(buf)))
    return None if n < 0 else buf.value.decode().split("\n")[:n]


class Plugin:
    """One plugin instance (create through the creator, or deserialize a blob)."""

    def __init__(self, handle):
        if not handle:
            raise ValueError("plugin creation failed")
        self.handle = C.c_void_p(handle)

    @classmethod
    def create(cls, plugin_name: str, fields: dict, layer_name="layer"):
        """fields: name -> numpy array (int32 or float32); passed as PluginFields with length 1, like the reference."""
        keep, arr = [], (PluginField * len(fields))()
        for i, (k, v) in enumerate(fields.items()):
            a = np.ascontiguousarray(v)
            keep.append(a)
            arr[i] = PluginField(k.encode(), a.ctypes.data, PF_FLOAT32 if a.dtype == np.float32 else PF_INT32, 1)
        return cls(_lib().sessd_plugin_create(plugin_name.encode(), layer_name.encode(), arr, len(fields)))

    @classmethod
    def deserialize(cls, plugin_name: str, blob: bytes):
        return cls(_lib().sessd_plugin_deserialize(plugin_name.encode(), blob, C.c_size_t(len(blob))))

    def clone(self):
        return Plugin(_lib().sessd_plugin_clone(self.handle))

    def type(self):
        return _lib().sessd_plugin_type(self.handle).decode()

    def version(self):
        return _lib().sessd_plugin_version(self.handle).decode()

    def nb_outputs(self):
        return _lib().sessd_plugin_nb_outputs(self.handle)

    def output_dims(self, index, inputs):
        arr = (TensorDesc * len(inputs))(*inputs)
        out = TensorDesc()
        rc = _lib().sessd_plugin_output_dims(self.handle, index, arr, len(inputs), C.byref(out))
        return None if rc else out

    def output_dtype(self, index, input_types):
        arr = (C.c_int32 * len(input_types))(*input_types)
        return _lib().sessd_plugin_output_dtype(self.handle, index, arr, len(input_types))

    def supports_format(self, pos, in_out, nb_inputs):
        arr = (TensorDesc * len(in_out))(*in_out)
        return bool(_lib().sessd_plugin_supports_format(self.handle, pos, arr, nb_inputs, len(in_out) - nb_inputs))

    def configure(self, inputs, outputs):
        a, b = (TensorDesc * len(inputs))(*inputs), (TensorDesc * len(outputs))(*outputs)
        _lib().sessd_plugin_configure(self.handle, a, len(inputs), b, len(outputs))

    def workspace_size(self, inputs, outputs):
        a, b = (TensorDesc * len(inputs))(*inputs), (TensorDesc * len(outputs))(*outputs)
        return int(_lib().sessd_plugin_workspace_size(self.handle, a, len(inputs), b, len(outputs)))

    def enqueue(self, input_desc, output_desc, inputs, outputs, workspace, stream):
        """inputs / outputs: torch CUDA tensors; workspace: torch uint8 tensor or None. Returns the plugin's int."""
        a, b = (TensorDesc * len(input_desc))(*input_desc), (TensorDesc * len(output_desc))(*output_desc)
        ip = (C.c_void_p * len(inputs))(*[t.data_ptr() for t in inputs])
        op = (C.c_void_p * len(outputs))(*[t.data_ptr() for t in outputs])
        ws = C.c_void_p(workspace.data_ptr()) if workspace is not None else None
        return _lib().sessd_plugin_enqueue(self.handle, a, b, ip, op, ws, C.c_void_p(stream))

    def serialize(self) -> bytes:
        n = int(_lib().sessd_plugin_serialization_size(self.handle))
        buf = C.create_string_buffer(n)
        _lib().sessd_plugin_serialize(self.handle, buf)
        return buf.raw

    def destroy(self):
        if self.handle:
            _lib().sessd_plugin_destroy(self.handle)
            self.handle = C.c_void_p()

    def __del__(self):
        try:
            self.destroy()
        except Exception:
            pass
