"""Operator entry points. Every op runs the sm_100a kernel on CUDA tensors and the PyTorch
reference on CPU tensors; there is no silent fallback on a GPU (a missing native library raises).
Ops that take part in training are ``torch.autograd.Function``s whose backward is also native."""
