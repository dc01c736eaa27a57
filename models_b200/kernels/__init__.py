from . import ops
from .build import KernelBuildError, build_library, load_library, loaded_libraries
from .ops import KernelError
