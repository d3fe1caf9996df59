"""Small host helpers kept from the reference (torchao/utils.py:81-85)."""
from functools import reduce
from math import gcd


def find_multiple(n: int, *args: int) -> int:
    """Smallest multiple of lcm(args) that is >= n (torchao/utils.py:81-85)."""
    k = reduce(lambda x, y: x * y // gcd(x, y), args + (1,))
    if n % k == 0:
        return n
    return n + k - (n % k)


# ----------------------------------------------------------------------------------------------
# unwrap_tensor_subclass — torchao/utils.py:113-165
# ----------------------------------------------------------------------------------------------
import torch  # noqa: E402
from torch.nn.utils import parametrize  # noqa: E402


class UnwrapTensorSubclass(torch.nn.Module):
    """Parametrization that stores a (nested) tensor subclass as the plain tensors it is made of
    (torchao/utils.py:113-143).  right_inverse() walks __tensor_flatten__ down to plain tensors and remembers, per
    level, the class, its metadata and the attribute names; forward() rebuilds the levels from the leaves up with
    __tensor_unflatten__.  A state_dict of the parametrized module then holds ordinary tensors only."""

    def right_inverse(self, tensor):
        assert type(tensor) is not torch.Tensor
        levels, leaves = [], []
        pending = [tensor]
        while pending:
            obj = pending.pop()
            names, meta = obj.__tensor_flatten__()
            levels.append((type(obj), meta, list(names)))
            for name in names:
                inner = getattr(obj, name)
                if type(inner) is torch.Tensor:
                    leaves.append(inner)
                else:
                    assert isinstance(inner, torch.Tensor)
                    pending.append(inner)
        self.rebuild_stack = levels
        return leaves

    def forward(self, *tensors):
        work = list(tensors)
        for cls, meta, names in reversed(self.rebuild_stack):
            n = len(names)
            parts = dict(zip(names, work[-n:]))
            work = work[n:]
            work.append(cls.__tensor_unflatten__(parts, meta, None, None))
        assert len(work) == 1
        return work[0]


def unwrap_tensor_subclass(model, filter_fn=None):
    """Replaces the tensor-subclass weight of every nn.Linear in `model` by a parametrization over its plain inner
    tensors (torchao/utils.py:145-165), so that the state_dict and torch.export / AOT compilation see plain tensors."""
    for _, child in model.named_children():
        w = getattr(child, "weight", None)
        if (isinstance(child, torch.nn.Linear) and isinstance(w, torch.Tensor) and type(w) is not torch.Tensor
                and type(w) is not torch.nn.Parameter):
            parametrize.register_parametrization(child, "weight", UnwrapTensorSubclass())
        unwrap_tensor_subclass(child)
    return model
