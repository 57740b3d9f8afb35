"""Benchmark programs: allreduce microbenchmarks (C++ and PyTorch), the layer-wise DNN
communication model, and synthetic DDP training of ResNet-50, VGG-19 and BERT-large."""
