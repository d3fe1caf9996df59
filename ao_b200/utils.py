"""Small host helpers kept from the reference (torchao/utils.py:81-85)."""
from functools import reduce
from math import gcd


def find_multiple(n: int, *args: int) -> int:
    """Smallest multiple of lcm(args) that is >= n (torchao/utils.py:81-85)."""
    k = reduce(lambda x, y: x * y // gcd(x, y), args + (1,))
    if n % k == 0:
        return n
    return n + k - (n % k)
