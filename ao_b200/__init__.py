"""ao_b200: B200-native (sm_100a) weight-only quantized linear behind torchao's Python API."""
from . import _cabi  # noqa: F401


def check_status(device=None) -> None:
    """Raises if a kernel on `device` (default: the current CUDA device) has reported a device-side failure - a
    bounded wait that ran out - since the workspace of the current stream was created.  Synchronises the stream.
    The kernels never hang and never trap: they leave a status word, and this is how a serving loop reads it."""
    import torch
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    status = _cabi.workspace_status(dev)
    if status != _cabi.AO_OK:
        raise _cabi.AoError(status, f"a kernel on {dev} reported")


__all__ = ["check_status"]
