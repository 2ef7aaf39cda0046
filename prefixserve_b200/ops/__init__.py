"""Python faces of the CUDA kernels.  Each checks shapes, dtypes and layout on
the host and raises ``KernelError`` instead of launching on arguments a kernel
was not written for."""

from .deferred import NormedRows, PendingProduct  # noqa: F401
from .kernels import (  # noqa: F401
    ACTIVATIONS,
    KernelError,
    act_mul,
    add_rmsnorm,
    attention,
    embedding,
    gated_linear,
    last_product,
    linear,
    pair_interleaved_order,
    qkv_rope_append,
    residual_add,
    rope_append,
    sample,
    sample_slots,
    scatter_words,
    step_prepare,
    silu_mul,
)
