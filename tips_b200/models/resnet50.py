"""ResNet-50 v1.5 for channels-last bf16 training.

The reference's evaluated workload is a TensorFlow ResNet-50 trained through its
collective mode (README.md:12); the model itself is not part of the reference.
Here all convolutions are the tcgen05 implicit-GEMM kernels (the 7x7 stem
through a padded 8-channel copy of the image), their epilogue produces the
batch statistics, the normalisation layers are the fused sm_100a
kernels (BN + residual + ReLU in one pass, forward and backward) and the loss is
the fused softmax cross-entropy.
"""
from __future__ import annotations

import torch
import torch.nn as nn

from ..ops.conv import Conv2d, conv2d_passthrough, supported as _conv_supported
from ..ops.norm import BatchNorm2d
from ..ops.linear import Linear
from ..ops.pool import MaxPool3x3S2, global_avg_pool
from ..ops.pointwise import softmax_cross_entropy


class LibraryBatchNorm2d(nn.Module):
    """Same call signature as the fused BatchNorm2d, built from library ops (cuDNN batch norm, separate add
    and ReLU kernels).  Used only by the library-floor benchmark arm."""

    def __init__(self, num_features, relu=False):
        super().__init__()
        self.bn = nn.BatchNorm2d(num_features)
        self.relu = relu
        self.weight = self.bn.weight

    def forward(self, x, residual=None):
        y = self.bn(x)
        if residual is not None:
            y = y + residual
        return torch.relu(y) if self.relu else y


_NORM = BatchNorm2d
_LIBRARY_CONV = False


def _conv(cin, cout, k, stride=1, padding=0):
    if _LIBRARY_CONV:
        return nn.Conv2d(cin, cout, k, stride=stride, padding=padding, bias=False)
    return Conv2d(cin, cout, k, stride=stride, padding=padding)


class _StatsArena:
    """One zeroed fp32 buffer per forward pass from which every conv + batch-norm pair takes its [2, C] slot for the
    epilogue statistics: one fill kernel per step instead of one per layer."""

    def __init__(self):
        self.buf = None
        self.off = 0

    def begin(self, floats: int, device) -> None:
        self.buf = torch.zeros(floats, dtype=torch.float32, device=device)
        self.off = 0

    def end(self) -> None:
        self.buf = None

    def take(self, channels: int, device) -> torch.Tensor:
        n = 2 * channels
        if self.buf is None or self.buf.device != device or self.off + n > self.buf.numel():
            return torch.zeros(2, channels, dtype=torch.float32, device=device)
        v = self.buf[self.off:self.off + n].view(2, channels)
        self.off += n
        return v


_ARENA = _StatsArena()


def _conv_bn(conv, bn, x, residual=None, passthrough=False):
    """bn(conv(x)) (+ residual, ReLU); in training the convolution's epilogue hands the batch statistics to the
    normalisation, which then needs no reduction pass of its own.  With `passthrough` the result is a pair
    (output, alias of x for the block's other branch): the gradients of the two uses of x are then summed inside
    the convolution's data-gradient kernel."""
    if (isinstance(conv, Conv2d) and isinstance(bn, BatchNorm2d) and bn.training
            and _conv_supported(x, conv.weight, conv.stride, conv.padding)):
        stats = _ARENA.take(conv.out_channels, x.device)
        if passthrough:
            y, alias = conv2d_passthrough(x, conv.weight, conv.stride, conv.padding, stats)
            return bn(y, residual=residual, stats=stats), alias
        return bn(conv(x, stats=stats), residual=residual, stats=stats)
    out = bn(conv(x), residual=residual)
    return (out, x) if passthrough else out


class Bottleneck(nn.Module):
    expansion = 4

    def __init__(self, cin, width, stride=1, downsample=False):
        super().__init__()
        cout = width * self.expansion
        self.conv1 = _conv(cin, width, 1)
        self.bn1 = _NORM(width, relu=True)
        self.conv2 = _conv(width, width, 3, stride=stride, padding=1)  # v1.5: the stride sits on the 3x3
        self.bn2 = _NORM(width, relu=True)
        self.conv3 = _conv(width, cout, 1)
        self.bn3 = _NORM(cout, relu=True)  # ReLU after the residual add, fused
        nn.init.zeros_(self.bn3.weight)
        self.down = None
        if downsample:
            self.down = nn.Sequential()
            self.down.add_module("conv", _conv(cin, cout, 1, stride=stride))
            self.down.add_module("bn", _NORM(cout, relu=False))

    def forward(self, x):
        out, x = _conv_bn(self.conv1, self.bn1, x, passthrough=True)
        identity = x if self.down is None else _conv_bn(self.down.conv, self.down.bn, x)
        out = _conv_bn(self.conv2, self.bn2, out)
        return _conv_bn(self.conv3, self.bn3, out, residual=identity)


class ResNet50(nn.Module):
    def __init__(self, num_classes=1000, layers=(3, 4, 6, 3), width=64):
        super().__init__()
        self._stat_floats = None  # size of the per-forward statistics arena, counted on first use
        self.conv1 = _conv(3, width, 7, stride=2, padding=3)
        self.bn1 = _NORM(width, relu=True)
        self.maxpool = nn.MaxPool2d(3, stride=2, padding=1) if _LIBRARY_CONV else MaxPool3x3S2()
        blocks = []
        cin = width
        for stage, n in enumerate(layers):
            w = width * (2 ** stage)
            for i in range(n):
                stride = 2 if (i == 0 and stage > 0) else 1
                blocks.append(Bottleneck(cin, w, stride, downsample=(i == 0)))
                cin = w * Bottleneck.expansion
        self.blocks = nn.Sequential(*blocks)
        # library arm: torch pooling and nn.Linear (cuBLAS); otherwise the pooling kernel and the tcgen05 GEMM
        self.avgpool = nn.AdaptiveAvgPool2d(1) if _LIBRARY_CONV else None
        self.fc = nn.Linear(cin, num_classes) if _LIBRARY_CONV else Linear(cin, num_classes)
        for m in self.modules():
            if isinstance(m, nn.Conv2d):
                nn.init.kaiming_normal_(m.weight, mode="fan_out", nonlinearity="relu")  # Conv2d does the same itself

    def forward(self, x):
        if self.training and x.is_cuda:
            if self._stat_floats is None:
                self._stat_floats = sum(2 * m.num_features for m in self.modules() if isinstance(m, BatchNorm2d))
            _ARENA.begin(self._stat_floats, x.device)
        try:
            x = self.maxpool(_conv_bn(self.conv1, self.bn1, x))
            x = self.blocks(x)
        finally:
            _ARENA.end()
        x = torch.flatten(self.avgpool(x), 1) if self.avgpool is not None else global_avg_pool(x)
        return self.fc(x)

    def loss(self, images, labels):
        return softmax_cross_entropy(self.forward(images), labels)


def resnet50(num_classes=1000, dtype=torch.bfloat16, device="cuda", library_norm=False, library_conv=None):
    """`library_norm` / `library_conv` build the library-floor arm (cuDNN batch norm and convolutions)."""
    global _NORM, _LIBRARY_CONV
    _NORM = LibraryBatchNorm2d if library_norm else BatchNorm2d
    _LIBRARY_CONV = library_norm if library_conv is None else library_conv
    try:
        m = ResNet50(num_classes)
    finally:
        _NORM = BatchNorm2d
        _LIBRARY_CONV = False
    m = m.to(device=device, dtype=dtype)
    return _channels_last(m, device)


def _channels_last(m, device):
    """Library convolutions want channels-last weights; the tcgen05 Conv2d keeps its own [C_out, R, S, C_in] layout."""
    if torch.device(device).type == "cuda":
        for mod in m.modules():
            if isinstance(mod, nn.Conv2d):
                mod.to(memory_format=torch.channels_last)
    return m


def tiny_resnet(num_classes=10, dtype=torch.bfloat16, device="cuda", width=16):
    """Same block structure with one block per stage; for smoke tests.  With width=64 every convolution has the
    channel counts of the full model and runs on the tcgen05 kernels; narrower widths use the library fallback."""
    m = ResNet50(num_classes, layers=(1, 1, 1, 1), width=width).to(device=device, dtype=dtype)
    return _channels_last(m, device)
