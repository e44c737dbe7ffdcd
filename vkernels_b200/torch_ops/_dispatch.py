"""Calling convention of the ops in this package: ops validate themselves.

Same contract as the reference's ``torch_ops/_dispatch.py:27-60``: an input the
fused path cannot take (CPU tensor, wrong dtype, shape outside the validated
envelope) raises :class:`OpNotEligible` - a routine outcome the caller may
catch; anything else (``TypeError`` for structurally wrong arguments,
``RuntimeError`` for an operational failure such as a missing native library)
is a bug or an environment problem and propagates.
"""

__all__ = ["OpNotEligible", "require", "same_gpu_contiguous"]


class OpNotEligible(ValueError, TypeError):
    """The fused kernel cannot run these inputs."""


def require(condition: bool, message: str) -> None:
    if not condition:
        raise OpNotEligible(message)


def same_gpu_contiguous(*tensors) -> None:
    """Eligibility floor: CUDA-resident, one device, contiguous."""
    require(tensors[0].is_cuda, "inputs must be CUDA-resident (there is no CPU path)")
    require(all(t.device == tensors[0].device for t in tensors), "inputs must share one GPU")
    require(all(t.is_contiguous() for t in tensors), "inputs must be contiguous")
