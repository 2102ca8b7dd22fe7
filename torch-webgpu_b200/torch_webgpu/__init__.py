"""torch_webgpu: the `webgpu` PyTorch device, served by hand-written sm_100a CUDA kernels.

Importing the package has the same side effects as the reference's
python/torch_webgpu/__init__.py:6-15: PrivateUse1 is renamed to "webgpu", the `torch.webgpu`
device module is registered, Tensor / Module / Storage / PackedSequence get their `.webgpu()`
and `.is_webgpu` members, and `webgpu_backend` is registered with torch.compile.  The native
extension is mandatory: if it cannot be loaded the import fails, there is no CPU fallback.
"""
import torch

from . import _C  # noqa: F401  (registers the guard, the allocator and every op)
from . import webgpu

torch.utils.rename_privateuse1_backend("webgpu")
torch._register_device_module("webgpu", webgpu)
torch.utils.generate_methods_for_privateuse1_backend(
    for_tensor=True,
    for_module=True,
    for_storage=True,
    for_packed_sequence=True,
)

from .compiler.webgpu_compiler import webgpu_backend  # noqa: E402

__all__ = ["webgpu_backend", "webgpu"]
