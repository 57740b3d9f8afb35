"""Model definitions used by the training benchmarks (random initial weights, synthetic
data): ResNet-50, VGG-19 and BERT-large. The reference ships no model code; these are the
workloads its integrations are meant for (DDP gradient allreduce)."""
from .resnet50 import resnet50  # noqa: F401
from .vgg19 import vgg19  # noqa: F401
from .bert_large import BertConfig, BertForMaskedLM, bert_large  # noqa: F401
