"""deuteron_b200: B200-native kernels behind the Deuteron compile/launch surface.

    from deuteron_b200 import compile_kernel, Options, LocalRunner
    compiled = compile_kernel('kernel.ir.json', arch='sm_100a', options=Options(contraction_precision='bf16x3'))
    with LocalRunner(0) as runner:
        result = runner.run_kernel(meta['kernels'][0], compiled)

Compute runs only in libdeuteron_b200.so (hand-written CUDA for sm_100a, see csrc/); build it with
`python -m deuteron_b200.csrc.build`. Importing the package does not need a GPU; launching does.
"""
from .build import Compilation, clear_cache, compile_kernel, compile_many
from .options import Options
from .runner import LocalRunner, argument_array, compare_outputs
from .native import CudaError, DeviceWaitError

__version__ = '0.1.0'
__all__ = ['Compilation', 'CudaError', 'DeviceWaitError', 'LocalRunner', 'Options', 'argument_array', 'clear_cache',
           'compare_outputs', 'compile_kernel', 'compile_many']
