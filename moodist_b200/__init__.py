"""moodist_b200: a Blackwell-native ``torch.distributed`` backend with the public API of moodist.

Exports mirror the reference package (``py/moodist/__init__.py:62-89``).
"""

from queue import Empty

from .version import __version__
from ._core import (
    MoodistProcessGroup,
    MoodistBackend,
    TcpStore,
    serialize,
    deserialize,
    cuda_copy,
    set_prefer_kernel_less,
)
from .allocator import (
    enable_cuda_allocator,
    enable_cpu_allocator,
    cpu_allocator_debug,
    cuda_allocator_stats,
    symmetric_pool,
)
from .utils.trace import enable_profiling
from .backend import find_process_group, create_moodist_backend, get_backend, PreferKernelLessContext
from .options import MoodistOptions, MoodistOptionsContext, install as _install_options
from .queue import Queue, TransactionContextManager
from .compile import compile_op

_install_options(MoodistProcessGroup)

__all__ = [
    "__version__",
    "MoodistProcessGroup",
    "MoodistBackend",
    "enable_profiling",
    "enable_cuda_allocator",
    "enable_cpu_allocator",
    "cpu_allocator_debug",
    "cuda_copy",
    "set_prefer_kernel_less",
    "TcpStore",
    "serialize",
    "deserialize",
    "Queue",
    "TransactionContextManager",
    "Empty",
    "find_process_group",
    "create_moodist_backend",
    "get_backend",
    "PreferKernelLessContext",
    "MoodistOptions",
    "MoodistOptionsContext",
    "compile_op",
    "symmetric_pool",
    "cuda_allocator_stats",
]
