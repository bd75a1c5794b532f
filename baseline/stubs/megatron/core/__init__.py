"""Stand-in for the parts of ``megatron.core`` the reference imports.

Megatron-core is not installed in this image.  The reference needs it for one
type annotation (``TransformerConfig``) and, at run time, for the parallel
state of the training job; both are provided here on top of
``torch.distributed`` so that the reference's code runs unmodified.
"""
from . import parallel_state  # noqa: F401
