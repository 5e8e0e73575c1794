"""dl4s_b200 — a B200 (sm_100a) back-end for the attention path of DL4S.

`cuda` mirrors DL4S's DeviceType / MemoryOperatorsType / EngineType boundary on
top of the C ABI of libdl4s_cuda.so; `layers` mirrors the transformer layers
that use it. Build the library with `python -m dl4s_b200.build`.
"""
from ._lib import ACT_GELU_SIGMOID, ACT_RELU, PREC_F16, PREC_F16_SPLIT, PREC_FP32, DL4SCudaError, EXPORTS, LIB_PATH  # noqa: F401
