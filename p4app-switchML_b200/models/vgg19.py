"""VGG-19 (configuration E, no batch norm), 143.7 M parameters, 86 % of them in the three
fully connected layers — the communication-bound member of the benchmark set. With
``fused_fc=True`` fc6 and fc7 compute their weight gradients with the tcgen05 GEMM whose
epilogue is fused with the cross-GPU reduction (ops/wgrad.py)."""
import torch
from torch import nn

from ..ops.wgrad import FusedWgradLinear

_CFG = [64, 64, "M", 128, 128, "M", 256, 256, 256, 256, "M", 512, 512, 512, 512, "M", 512, 512, 512, 512, "M"]


class VGG19(nn.Module):
    def __init__(self, num_classes=1000, fused_fc=False):
        super().__init__()
        layers, c = [], 3
        for v in _CFG:
            if v == "M":
                layers.append(nn.MaxPool2d(2, 2))
            else:
                layers += [nn.Conv2d(c, v, 3, padding=1), nn.ReLU(inplace=True)]
                c = v
        self.features = nn.Sequential(*layers)
        lin = FusedWgradLinear if fused_fc else nn.Linear
        self.fc6 = lin(512 * 7 * 7, 4096)
        self.fc7 = lin(4096, 4096)
        self.fc8 = nn.Linear(4096, num_classes)
        self.relu = nn.ReLU(inplace=True)
        self.drop = nn.Dropout(0.5)

    def fused_layers(self):
        return [m for m in (self.fc6, self.fc7) if isinstance(m, FusedWgradLinear)]

    def forward(self, x):
        x = torch.flatten(self.features(x), 1)
        x = self.drop(self.relu(self.fc6(x)))
        x = self.drop(self.relu(self.fc7(x)))
        return self.fc8(x)


def vgg19(num_classes=1000, fused_fc=False):
    return VGG19(num_classes, fused_fc)
