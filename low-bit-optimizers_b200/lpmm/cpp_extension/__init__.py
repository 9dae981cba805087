"""Stand-ins for the reference's two compiled extension modules, under the same import paths
(``lpmm.cpp_extension.fused_adamw``, ``lpmm.cpp_extension.quantization``) and with the same
function signatures, implemented on the C-ABI CUDA library."""
