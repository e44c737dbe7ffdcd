"""B200-native fused MXFP4 mixture-of-experts layer.

``vkernels_b200.torch_ops``   torch-tensor ops over the C ABI
``vkernels_b200.experts``     layer object with persistent scratch (serving call sequence)
``vkernels_b200.dist``        expert-parallel layer over torch.distributed (NCCL)
``vkernels_b200.synthetic``   seeded workloads of the benchmark configurations
``vkernels_b200.build``       in-tree nvcc build of libvkernels_b200.so
"""
__version__ = "0.1.0"
