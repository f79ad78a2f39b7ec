"""Frame -> boxes: the reference's whole network (se-ssd-ai-trt.cpp:1138-1440) around this package's kernels.

The sparse front end (voxelise, 14 sparse layers, dense BEV map with its zero border) and the post-processing
(anchor decoding, score filter, rotated NMS) are the library's CUDA kernels. The 2D neck and head between them
are plain dense convolutions, which the reference leaves to TensorRT's own layers (`addConvolutionNd`,
`addDeconvolutionNd`, `addScale`, `addSoftMax`, :1262-1374); here they are torch's convolution calls in fp16
with the batch norms folded in: library glue, as in the reference. Needs a CUDA device."""
from __future__ import annotations

import numpy as np

from . import schedule, synth

# (name, conv blob prefix, batch-norm blob prefix, cin, cout, ksize, stride, padding): se-ssd-ai-trt.cpp:1262-1306
# with the sizes of params.h (BOTTOM_UP_BLOCK_*, TRANS_*, DECONV_BLOCK_*, CONV_*, W_*).
NECK_LAYERS = (
    ("bu0_0", "neck.bottom_up_block_0.1", "neck.bottom_up_block_0.2", 128, 128, 3, 1, 0),   # runs on the padded map
    ("bu0_1", "neck.bottom_up_block_0.4", "neck.bottom_up_block_0.5", 128, 128, 3, 1, 1),
    ("bu0_2", "neck.bottom_up_block_0.7", "neck.bottom_up_block_0.8", 128, 128, 3, 1, 1),
    ("bu1_0", "neck.bottom_up_block_1.0", "neck.bottom_up_block_1.1", 128, 256, 3, 2, 1),
    ("bu1_1", "neck.bottom_up_block_1.3", "neck.bottom_up_block_1.4", 256, 256, 3, 1, 1),
    ("bu1_2", "neck.bottom_up_block_1.6", "neck.bottom_up_block_1.7", 256, 256, 3, 1, 1),
    ("trans_0", "neck.trans_0.0", "neck.trans_0.1", 128, 128, 1, 1, 0),
    ("trans_1", "neck.trans_1.0", "neck.trans_1.1", 256, 256, 1, 1, 0),
    ("deconv_0", "neck.deconv_block_0.0", "neck.deconv_block_0.1", 256, 128, 3, 2, 1),      # transposed, output padding 1
    ("deconv_1", "neck.deconv_block_1.0", "neck.deconv_block_1.1", 256, 128, 3, 2, 1),
    ("conv_0", "neck.conv_0.0", "neck.conv_0.1", 128, 128, 3, 1, 1),
    ("conv_1", "neck.conv_1.0", "neck.conv_1.1", 128, 128, 3, 1, 1),
    ("w_0", "neck.w_0.0", "neck.w_0.1", 128, 1, 1, 1, 0),                                   # batch norm, no ReLU
    ("w_1", "neck.w_1.0", "neck.w_1.1", 128, 1, 1, 1, 0),
)
# (name, blob prefix, cout): 1x1 convolutions with bias, se-ssd-ai-trt.cpp:1341-1377
HEAD_LAYERS = (
    ("box", "bbox_head.tasks.0.conv_box", 14),
    ("cls", "bbox_head.tasks.0.conv_cls", 2),
    ("iou", "bbox_head.tasks.0.conv_iou", 2),
    ("dir", "bbox_head.tasks.0.conv_dir", 4),
)
BN2D_EPS = 1e-5   # addBatchNorm2d is called with 1e-5 everywhere (se-ssd-ai-trt.cpp:1055)


def random_neck_weights(seed=0x5E55D000 + 400):
    """Seeded random-init blobs under the reference's state-dict names (no trained weights are available):
    He-scaled convolutions, batch norms near identity, small head biases."""
    blobs = {}
    for i, (name, conv, bn, cin, cout, k, _s, _p) in enumerate(NECK_LAYERS):
        shape = (cin, cout, k, k) if name.startswith("deconv") else (cout, cin, k, k)
        fan_in = cin * k * k / (4.0 if name.startswith("deconv") else 1.0)   # a stride-2 transposed conv sees a quarter of the taps
        blobs[conv + ".weight"] = synth.normal_f32(seed + 31 * i, shape, float(np.sqrt(2.0 / fan_in)))
        s = synth.Stream(seed + 31 * i + 5)
        blobs[bn + ".weight"] = (1.0 + 0.05 * s.normal(cout)).astype(np.float32)
        blobs[bn + ".bias"] = (0.02 * s.normal(cout)).astype(np.float32)
        blobs[bn + ".running_mean"] = (0.02 * s.normal(cout)).astype(np.float32)
        blobs[bn + ".running_var"] = (1.0 + 0.1 * s.uniform(cout)).astype(np.float32)
    for i, (name, prefix, cout) in enumerate(HEAD_LAYERS):
        blobs[prefix + ".weight"] = synth.normal_f32(seed + 1000 + 31 * i, (cout, 128, 1, 1), 0.05)
        blobs[prefix + ".bias"] = synth.normal_f32(seed + 1000 + 31 * i + 5, (cout,), 0.01)
    return blobs


class Neck2D:
    """The BEV neck and head (se-ssd-ai-trt.cpp:1262-1440) as fp16 torch convolutions on the GPU.
    `blobs`: {state-dict name: array}, e.g. formats.Wts contents or random_neck_weights()."""

    def __init__(self, blobs, device="cuda"):
        import torch

        from .formats import fold_batchnorm

        if not torch.cuda.is_available():
            raise RuntimeError("Neck2D needs a CUDA device")
        self.torch, self.device = torch, device
        self.w, self.b = {}, {}
        for name, conv, bn, cin, cout, k, _s, _p in NECK_LAYERS:
            w = np.asarray(blobs[conv + ".weight"], np.float32)
            transposed = name.startswith("deconv")
            w = w.reshape((cin, cout, k, k) if transposed else (cout, cin, k, k))
            scale, shift = fold_batchnorm(*[blobs[bn + s] for s in (".weight", ".bias", ".running_mean", ".running_var")],
                                          BN2D_EPS)
            w = w * (scale[None, :, None, None] if transposed else scale[:, None, None, None])
            self.w[name] = torch.from_numpy(np.ascontiguousarray(w)).to(device).half().contiguous(memory_format=torch.channels_last)
            self.b[name] = torch.from_numpy(shift).to(device).half()
        # the four heads read the same map: one convolution with 22 output channels
        hw = np.concatenate([np.asarray(blobs[p + ".weight"], np.float32).reshape(c, 128, 1, 1) for _, p, c in HEAD_LAYERS])
        hb = np.concatenate([np.asarray(blobs[p + ".bias"], np.float32).reshape(c) for _, p, c in HEAD_LAYERS])
        self.head_w = torch.from_numpy(hw).to(device).half().contiguous(memory_format=torch.channels_last)
        self.head_b = torch.from_numpy(hb).to(device).half()

    def _conv(self, x, name, relu=True):
        F = self.torch.nn.functional
        _n, _c, _b, _cin, _cout, _k, s, p = next(l for l in NECK_LAYERS if l[0] == name)
        if name.startswith("deconv"):
            y = F.conv_transpose2d(x, self.w[name], self.b[name], stride=s, padding=p, output_padding=1)
        else:
            y = F.conv2d(x, self.w[name], self.b[name], stride=s, padding=p)
        return F.relu_(y) if relu else y

    def features(self, bev_padded):
        """[B, 128, 202, 178] fp16 (the zero-padded BEV map) -> fused neck output [B, 128, 200, 176]."""
        torch = self.torch
        x = bev_padded.contiguous(memory_format=torch.channels_last)
        for n in ("bu0_0", "bu0_1", "bu0_2"):
            x = self._conv(x, n)
        x0 = x
        for n in ("bu1_0", "bu1_1", "bu1_2"):
            x = self._conv(x, n)
        t0, t1 = self._conv(x0, "trans_0"), self._conv(x, "trans_1")
        o0 = self._conv(self._conv(t1, "deconv_0") + t0, "conv_0")
        o1 = self._conv(self._conv(t1, "deconv_1"), "conv_1")
        w = torch.softmax(torch.cat([self._conv(o0, "w_0", relu=False), self._conv(o1, "w_1", relu=False)], dim=1).float(),
                          dim=1).half()
        return o0 * w[:, 0:1] + o1 * w[:, 1:2]

    def __call__(self, bev_padded):
        """-> dict of fp32 head outputs in the layout the post-processing plugins take:
        box [B, 70400, 7], cls [B, 70400, 1], iou [B, 70400, 1], dir [B, 70400, 2] (anchor = (y*W + x)*2 + a)."""
        F = self.torch.nn.functional
        y = F.conv2d(self.features(bev_padded), self.head_w, self.head_b).permute(0, 2, 3, 1).float()   # [B, H, W, 22]
        B = y.shape[0]
        out, c0 = {}, 0
        for name, _p, c in HEAD_LAYERS:
            out[name] = y[..., c0:c0 + c].reshape(B, -1, c // 2).contiguous()
            c0 += c
        return out


class Detector:
    """points -> kept boxes, the reference's per-frame loop body (se-ssd-ai-trt.cpp:1858-1892) on the device."""

    def __init__(self, backbone, neck: Neck2D, score_threshold=schedule.SCORE_THRESHOLD, nms_thresh=schedule.NMS_THRESH,
                 max_box_num=schedule.MAX_BOX_NUM):
        from . import anchor_params, filter_params

        self.backbone, self.neck = backbone, neck
        backbone.set_padding(1, 1, 1, 1)                      # ZERO_PADDING_2D_* of params.h, folded into the BEV write
        self.anchors = anchor_params()
        self.filter = filter_params(max_box_num=max_box_num, score_threshold=score_threshold)
        self.nms_thresh = nms_thresh

    def capture(self, max_points, batch=1):
        """Records the whole chain for `batch` frames of up to `max_points` points into one CUDA graph (every
        enqueue call of the library is capturable: no allocation, no synchronisation, all counts read on the
        device). Afterwards replay(points, sizes) costs one graph launch instead of some sixty kernel launches."""
        import torch

        from . import filter_boxes, rotated_nms

        bb = self.backbone
        self._pts = torch.zeros((batch, max_points, 4), device="cuda")
        self._sizes = torch.zeros((batch,), dtype=torch.int32, device="cuda")
        self._ws = torch.empty(bb.workspace_bytes(batch, max_points), dtype=torch.uint8, device="cuda")
        self._bev = torch.empty(bb.dense_shape(batch), dtype=torch.float16, device="cuda")

        def chain():
            bb.run(self._pts, self._sizes, self._ws, self._bev)
            heads = self.neck(self._bev)
            flt = filter_boxes(heads["box"], heads["cls"], heads["iou"], heads["dir"], self.filter, anchors=self.anchors,
                               read_back_status=False)
            boxes, num = rotated_nms(flt["box"], flt["valid"], self.nms_thresh)
            return dict(boxes=boxes, num=num, heads=heads, filtered=flt)

        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(3):              # kernel attributes, convolution plans and allocator pools settle here
                chain()
        side.synchronize()
        self._graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self._graph, stream=side):
            self._out = chain()
        return self

    def replay(self, points, sizes, read_back_status=True):
        """points f32 [B, P, 4] and sizes i32 [B] (device or pinned host tensors) -> the captured outputs, which
        are overwritten by the next replay."""
        from . import read_status

        self._pts.copy_(points, non_blocking=True)
        self._sizes.copy_(sizes, non_blocking=True)
        self._graph.replay()
        out = dict(self._out)
        if read_back_status:
            out["status"] = read_status(self._ws) | read_status(self._out["filtered"]["workspace"])
        return out

    def __call__(self, points, sizes):
        """points cuda f32 [B, P, 4], sizes cuda i32 [B] -> dict(boxes [B, M, 9], num [B], heads, filtered, status)."""
        from . import filter_boxes, read_status, rotated_nms

        bev, ws = self.backbone.run(points, sizes)
        heads = self.neck(bev)
        filtered = filter_boxes(heads["box"], heads["cls"], heads["iou"], heads["dir"], self.filter, anchors=self.anchors)
        boxes, num = rotated_nms(filtered["box"], filtered["valid"], self.nms_thresh)
        return dict(boxes=boxes, num=num, heads=heads, filtered=filtered,
                    status=read_status(ws) | filtered["status"])
