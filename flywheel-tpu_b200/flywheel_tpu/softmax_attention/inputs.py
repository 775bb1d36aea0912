"""Argument checks shared by the entry points; the exception types and
messages follow flywheel_tpu/softmax_attention/inputs.py:61-87, 218-251 of the
reference project."""

from flywheel_tpu.softmax_attention import _arrays


def check_common_kwargs(window_size, dropout_p=0.0, softcap=0.0,
                        alibi_slopes=None, deterministic=False,
                        return_attn_probs=False):
    if dropout_p != 0.0:
        raise NotImplementedError("dropout_p is not supported.")
    window_size = tuple(window_size)
    if len(window_size) != 2 or any(
        bound != -1 and bound < 0 for bound in window_size
    ):
        raise ValueError(
            "window_size must be a 2-tuple of -1 (unbounded) or non-negative"
            f" ints; got {window_size}."
        )
    if softcap < 0.0:
        raise ValueError(f"softcap must be non-negative; got {softcap}.")
    if alibi_slopes is not None:
        raise NotImplementedError("alibi_slopes is not supported.")
    if deterministic:
        raise NotImplementedError(
            "deterministic is not supported; the forward kernel is"
            " deterministic already."
        )
    if return_attn_probs:
        raise NotImplementedError("return_attn_probs is not supported.")
    return window_size


def resolve_window(window_size, causal):
    """(left, right) reach around the bottom-right diagonal, None unbounded;
    causal forces right to 0 (variant.py:205-217 of the reference)."""
    left = None if window_size[0] == -1 else window_size[0]
    if causal:
        right = 0
    elif window_size[1] == -1:
        right = None
    else:
        right = window_size[1]
    return left, right


def check_paged_window(window, window_size):
    if window[1] not in (None, 0):
        raise NotImplementedError(
            "a paged KV cache takes a window right bound of -1 (unbounded)"
            f" or 0 (causal) only; got window_size={window_size}."
        )


def descale_operand(descale, arg_name, device):
    """One per-tensor KV descale as a device f32 scalar (it may live on the
    device already: a new value needs no new kernel); None is 1."""
    if descale is None:
        return None
    tensor = _arrays.to_device(descale, device, dtype="float32")
    if tensor.numel() != 1:
        raise ValueError(
            f"{arg_name} must be one per-tensor value; got shape"
            f" {tuple(tensor.shape)}."
        )
    return tensor.reshape(1)


def sinks_operand(sinks, nheads, device):
    """sinks as a (nheads,) float32 device array, or None."""
    if sinks is None:
        return None
    shape = tuple(_arrays.shape(sinks))
    if shape != (nheads,) or not _arrays.is_floating(sinks):
        raise ValueError(
            f"learnable_sink must be a ({nheads},) float array, one logit per"
            f" query head; got {shape} {_arrays.dtype_name(_arrays.dtype(sinks))}."
        )
    return _arrays.to_device(sinks, device, dtype="float32").contiguous()
