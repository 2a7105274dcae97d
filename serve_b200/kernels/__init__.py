from .build import BuildError, build_library, build_many  # noqa: F401
from .cuda import CudaKernels, KernelError, all_jobs, attention_job, core_jobs, load_kernels  # noqa: F401
