"""Operator layer: autograd functions over the sm_100a kernels, with plain PyTorch fp32/CPU restatements
of the same math used on machines without a GPU and as numerical references in the tests."""
