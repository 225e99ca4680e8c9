"""Byte counters for host<->device traffic issued by the framework itself (prompt / batch uploads, token and
log-prob read-backs).  The benchmark reports them per step."""
_H2D = 0
_D2H = 0


def add_h2d(n: int):
    global _H2D
    _H2D += int(n)


def add_d2h(n: int):
    global _D2H
    _D2H += int(n)


def tensor_bytes(*ts) -> int:
    return sum(t.numel() * t.element_size() for t in ts if t is not None)


def reset():
    global _H2D, _D2H
    _H2D = _D2H = 0


def get():
    return _H2D, _D2H
