"""B200 (sm_100a) kernels for Linnet's weight-only quantized linear layers.

The package mirrors the pieces of the reference that this hot path consists of:

* `kernels`    - the torch operators `linnet::int4_linear`, `linnet::gemv8`,
                 `linnet::w8a16` and `dequantize8` (reference:
                 python/linnet/src/linnet/torch/kernels.py)
* `quantized`  - `int8_operands` / `int8_linear` / `int8_group_*` (reference:
                 python/linnet/src/linnet/torch/quantized.py)
* `int4`       - `_int4_pack` / `_int4_linear` / `_int4_weight`, the helpers the
                 reference's generated source defines (src/backend/torch_source.cpp:1482-1570)
* `quant`      - `quantize_int4_groups` / `quantize_int8_groups` / `pack_int4_groups`
                 on the GPU (reference: python/linnet/src/linnet/quant.py)
* `install`    - makes a process that uses `linnet.torch.load` dispatch to the above
* `decoder`    - a Llama-3.1-8B-shaped tensor-parallel int4 decoder used for the
                 decode benchmark

Every operator calls hand-written CUDA through the C ABI of `include/b200q.h`;
nothing here falls back to PyTorch arithmetic or to a CPU.
"""

from ._lib import B200QError, load as load_library  # noqa: F401

__all__ = ["B200QError", "load_library"]
