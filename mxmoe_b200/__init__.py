"""mxmoe_b200: B200 (sm_100a) mixed-precision MoE grouped GEMM behind the operator API of MxMoE.

Sub-modules
-----------
``ops``       drop-in for the reference's ``mxmoe_ops`` pybind module
``gg``        grouped-GEMM launcher (problem lists, prepared workspaces)
``layer``     host-sync-free MoE layer pipeline (routing -> quantise -> GEMMs -> combine)
``ep``        expert-parallel layer over ``torch.distributed`` (NCCL all-to-all)
``weights``   offline weight quantisation and packing in the reference's layouts
``workload``  seeded synthetic layers of the benchmark configurations
``build``     nvcc build of ``libmxmoe_b200.so``

The compute path lives in ``libmxmoe_b200.so`` (C ABI: ``include/mxmoe_b200.h``);
importing the package does not load it, the first operator call does, and it
raises if the library is missing - there is no CPU or PyTorch fallback.
"""
__version__ = "0.1.0"
