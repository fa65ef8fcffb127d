from .ops import CudaOps, KernelError
