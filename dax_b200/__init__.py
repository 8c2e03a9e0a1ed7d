"""dax_b200: B200-native (sm_100a) implementation of DAX's Ulysses self-attention hot path.

Sub-packages mirror the reference's layout: ``quant`` (dynamic INT8/FP8 linears and the module
swap), ``parallel`` (Ulysses sequence parallelism), ``adapters.wan`` (the attention processor and
``optimize_pipe``).  The kernels live in ``libdax_b200.so`` (``dax_b200/csrc``, C ABI in
``include/dax_b200.h``); ``dax_b200.ops`` wraps them for torch tensors."""
__version__ = "0.1.0"
