"""Test infrastructure: the reference's 2D neck and head (se-ssd-ai-trt.cpp:1262-1440) restated layer by layer
in fp32 on the CPU, the checker for the fp16 GPU glue in the package's detector module. Only tests import this.
parity unpinned: the reference ships neither trained weights nor recorded activations; the layer graph, the
batch-norm arithmetic and the output reshapes are restated from its network builder."""
from __future__ import annotations

import numpy as np
import torch
import torch.nn.functional as F


def _bn(x, blobs, prefix, eps=1e-5):
    """addBatchNorm2d (se-ssd-ai-trt.cpp:1013-1043): a per-channel scale layer, y = x * scale + shift."""
    g, b, m, v = (torch.from_numpy(np.asarray(blobs[prefix + s], np.float32))
                  for s in (".weight", ".bias", ".running_mean", ".running_var"))
    scale = g / torch.sqrt(v + eps)
    shift = b - m * g / torch.sqrt(v + eps)
    return x * scale[None, :, None, None] + shift[None, :, None, None]


def _w(blobs, name, shape):
    return torch.from_numpy(np.asarray(blobs[name], np.float32).reshape(shape).copy())


def conv_bn(x, blobs, conv, bn, cin, cout, k, s, p, relu=True):
    """convBnLELU / convBn (se-ssd-ai-trt.cpp:1046-1078): convolution without bias, batch norm, ReLU (the
    alpha the builder sets is ignored by a plain ReLU activation)."""
    y = _bn(F.conv2d(x, _w(blobs, conv + ".weight", (cout, cin, k, k)), None, stride=s, padding=p), blobs, bn)
    return F.relu(y) if relu else y


def deconv_bn(x, blobs, conv, bn, cin, cout, k=3, s=2, p=1):
    """deconvBnLELU (se-ssd-ai-trt.cpp:1080-1100): transposed convolution, stride 2, pre-padding 1 and no
    post-padding, i.e. output size 2 * input; in torch terms padding 1 with output_padding 1."""
    y = F.conv_transpose2d(x, _w(blobs, conv + ".weight", (cin, cout, k, k)), None, stride=s, padding=p, output_padding=1)
    return F.relu(_bn(y, blobs, bn))


def neck_and_head(bev_padded, blobs):
    """bev_padded: float32 array [B, 128, 202, 178] -> dict of float32 arrays box [B, 70400, 7], cls, iou
    [B, 70400, 1], dir [B, 70400, 2], plus `features` [B, 128, 200, 176]."""
    with torch.no_grad():
        x = torch.from_numpy(np.asarray(bev_padded, np.float32))
        n = "neck.bottom_up_block_0."
        x = conv_bn(x, blobs, n + "1", n + "2", 128, 128, 3, 1, 0)          # :1262-1271, on the zero-padded map
        x = conv_bn(x, blobs, n + "4", n + "5", 128, 128, 3, 1, 1)
        x0 = conv_bn(x, blobs, n + "7", n + "8", 128, 128, 3, 1, 1)
        n = "neck.bottom_up_block_1."
        x = conv_bn(x0, blobs, n + "0", n + "1", 128, 256, 3, 2, 1)         # :1272-1281
        x = conv_bn(x, blobs, n + "3", n + "4", 256, 256, 3, 1, 1)
        x1 = conv_bn(x, blobs, n + "6", n + "7", 256, 256, 3, 1, 1)
        t0 = conv_bn(x0, blobs, "neck.trans_0.0", "neck.trans_0.1", 128, 128, 1, 1, 0)      # :1282-1285
        t1 = conv_bn(x1, blobs, "neck.trans_1.0", "neck.trans_1.1", 256, 256, 1, 1, 0)
        d0 = deconv_bn(t1, blobs, "neck.deconv_block_0.0", "neck.deconv_block_0.1", 256, 128) + t0   # :1286-1288
        d1 = deconv_bn(t1, blobs, "neck.deconv_block_1.0", "neck.deconv_block_1.1", 256, 128)        # :1289-1290
        o0 = conv_bn(d0, blobs, "neck.conv_0.0", "neck.conv_0.1", 128, 128, 3, 1, 1)
        o1 = conv_bn(d1, blobs, "neck.conv_1.0", "neck.conv_1.1", 128, 128, 3, 1, 1)
        w0 = conv_bn(o0, blobs, "neck.w_0.0", "neck.w_0.1", 128, 1, 1, 1, 0, relu=False)     # :1295-1298
        w1 = conv_bn(o1, blobs, "neck.w_1.0", "neck.w_1.1", 128, 1, 1, 1, 0, relu=False)
        w = torch.softmax(torch.cat([w0, w1], dim=1), dim=1)                                  # :1299-1303
        feat = o0 * w[:, 0:1] + o1 * w[:, 1:2]                                                # :1304-1316
        out = {"features": feat.numpy()}
        B = feat.shape[0]
        for name, prefix, cout in (("box", "bbox_head.tasks.0.conv_box", 14), ("cls", "bbox_head.tasks.0.conv_cls", 2),
                                   ("iou", "bbox_head.tasks.0.conv_iou", 2), ("dir", "bbox_head.tasks.0.conv_dir", 4)):
            y = F.conv2d(feat, _w(blobs, prefix + ".weight", (cout, 128, 1, 1)), _w(blobs, prefix + ".bias", (cout,)))
            # shuffle to [B, H, W, C], then reshape to [B, H*W*2, C/2]   (:1345-1408)
            out[name] = y.permute(0, 2, 3, 1).reshape(B, -1, cout // 2).contiguous().numpy()
        return out
