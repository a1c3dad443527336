"""O(3)/SO(3) irrep bookkeeping for the tensor-product path.

Host-side metadata only: nothing here touches the GPU.  The public surface
(names, constructor forms, iteration order, string format) follows
``equitorch/irreps/__init__.py`` of the reference so that table builders and
modules written against it keep working:

* ``Irrep(l, p)`` / ``Irrep("2e")`` / ``Irrep(1)``      (reference :12-158)
* ``Irreps("6x0+1+2e")`` / ``Irreps((0, 3))`` / lists    (reference :240-838)
* iteration and ``len`` are multiplicity-expanded        (reference :558-584)
* ``has_path``, ``check_irreps``, ``irrep_segments`` …   (reference :213-238, :889-974)
"""
from __future__ import annotations

import math
import re
from functools import reduce
from typing import Dict, Iterable, Iterator, List, Sequence, Tuple, Union

import torch

_PARITY = {"e": 1, "o": -1, 1: 1, -1: -1, 0: 0, None: 0}
_TERM = re.compile(r"(?:(\d+)x)?(\d+)([eo]?)")


class Irrep:
    """One irrep: degree ``l`` and parity ``p`` in {+1 ('e'), -1 ('o'), 0 (SO(3))}."""

    __slots__ = ("l", "p")

    def __init__(self, *spec):
        if len(spec) == 1 and isinstance(spec[0], tuple):
            spec = spec[0]
        if len(spec) == 1:
            (a,) = spec
            if isinstance(a, Irrep):
                l, p = a.l, a.p
            elif isinstance(a, str):
                m = _TERM.fullmatch(a.strip())
                if m is None or m.group(1):
                    raise ValueError(f"cannot parse irrep {a!r}")
                l, p = int(m.group(2)), (m.group(3) or None)
            elif isinstance(a, int):
                l, p = a, None
            else:
                raise TypeError(f"cannot build an Irrep from {type(a).__name__}")
        elif len(spec) == 2:
            l, p = spec
            if not isinstance(l, int) or p is None:
                raise TypeError("two-argument form is Irrep(l:int, p)")
        else:
            raise TypeError("Irrep takes (l), (l, p), ('2e') or ((l, p))")
        if p not in _PARITY:
            raise ValueError("parity must be 'e', 'o', +1, -1, 0 or None")
        if not isinstance(l, int) or l < 0:
            raise ValueError("l must be a non-negative integer")
        self.l = l
        self.p = _PARITY[p]

    @property
    def dim(self) -> int:
        return 2 * self.l + 1

    def __iter__(self):
        yield self.l
        yield self.p

    def __repr__(self) -> str:
        return f"{self.l}{'' if self.p == 0 else 'e' if self.p > 0 else 'o'}"

    def __hash__(self) -> int:
        return hash((self.l, self.p))

    def __eq__(self, other) -> bool:
        if isinstance(other, str):
            return repr(self) == other
        if isinstance(other, int):
            return self.p == 0 and self.l == other
        if isinstance(other, (Irrep, tuple)):
            l, p = other
            return self.l == int(l) and self.p == _PARITY[p]
        return False

    def __mul__(self, other: "Irrep") -> "Irreps":
        """Selection rule |l1-l2| <= l <= l1+l2, parity multiplies (reference :125-158)."""
        if not isinstance(other, Irrep):
            raise TypeError(f"Irrep * {type(other).__name__} is undefined")
        return Irreps([Irrep(l, self.p * other.p)
                       for l in range(abs(self.l - other.l), self.l + other.l + 1)])


def parse_irreps(text: str) -> List[Tuple[Irrep, int]]:
    """``'6x0+1+2e'`` -> ``[(0, 6), (1, 1), (2e, 1)]``."""
    groups = []
    for term in text.replace(" ", "").split("+"):
        if not term:
            continue
        m = _TERM.fullmatch(term)
        if m is None:
            raise ValueError(f"Invalid term: {term}")
        mul = int(m.group(1)) if m.group(1) else 1
        if mul < 1:
            raise ValueError(f"Multiplicity must be >=1 in '{term}'")
        groups.append((Irrep(m.group(2) + m.group(3)), mul))
    return groups


def show_irreps(groups: Sequence[Tuple[Irrep, int]]) -> str:
    return "+".join((f"{mul}x" if mul != 1 else "") + repr(ir) for ir, mul in groups)


class Irreps:
    """Ordered direct sum of irreps with multiplicities (``irrep_groups``)."""

    def __init__(self, spec: Union[str, tuple, list, Irrep, "Irreps"]):
        if isinstance(spec, Irreps):
            groups = list(spec.irrep_groups)
        elif isinstance(spec, str):
            groups = parse_irreps(spec)
        elif isinstance(spec, Irrep):
            groups = [(spec, 1)]
        elif isinstance(spec, tuple):
            if len(spec) == 2 and all(isinstance(v, int) for v in spec):
                groups = [(Irrep(l), 1) for l in range(spec[0], spec[1] + 1)]
            elif len(spec) == 2 and isinstance(spec[0], Irrep) and isinstance(spec[1], int):
                groups = [spec]
            else:
                raise ValueError("tuple form is (l_min, l_max) or (Irrep, mul)")
        elif isinstance(spec, list):
            groups = []
            for item in spec:
                if isinstance(item, Irrep):
                    groups.append((item, 1))
                elif isinstance(item, tuple) and isinstance(item[0], Irrep):
                    groups.append((item[0], item[1]))
                else:
                    groups.append((Irrep(item), 1))
        else:
            raise TypeError(f"cannot build Irreps from {type(spec).__name__}")
        self.irrep_groups: List[Tuple[Irrep, int]] = groups

    # ---- constructors -------------------------------------------------
    @staticmethod
    def spherical_harmonics(max_degree: int, parity_even_degree="e") -> "Irreps":
        if parity_even_degree not in ("e", "o"):
            raise ValueError("parity_even_degree must be 'e' or 'o'")
        flip = {"e": "o", "o": "e"}
        return Irreps([f"{l}{parity_even_degree if l % 2 == 0 else flip[parity_even_degree]}"
                       for l in range(max_degree + 1)])

    @staticmethod
    def both_parities(max_degree: int, min_degree: int = 0) -> "Irreps":
        return Irreps([Irrep(l, p) for l in range(min_degree, max_degree + 1) for p in ("e", "o")])

    # ---- sequence protocol (multiplicity expanded) ---------------------
    def __iter__(self) -> Iterator[Irrep]:
        for ir, mul in self.irrep_groups:
            for _ in range(mul):
                yield ir

    def __len__(self) -> int:
        return sum(mul for _, mul in self.irrep_groups)

    def __getitem__(self, index):
        flat = list(self)
        if isinstance(index, int):
            if not -len(flat) <= index < len(flat):
                raise IndexError("Irrep index out of range")
            return flat[index]
        if isinstance(index, slice):
            if index.indices(len(flat))[2] != 1:
                raise ValueError("Irreps slicing only supports a step of 1")
            return Irreps(flat[index])
        raise TypeError(f"Irreps indices must be integers or slices, not {type(index).__name__}")

    def dims(self) -> Iterator[int]:
        for ir in self:
            yield ir.dim

    @property
    def dim(self) -> int:
        return sum(ir.dim * mul for ir, mul in self.irrep_groups)

    @property
    def l_max(self) -> int:
        return max(ir.l for ir, _ in self.irrep_groups)

    # ---- text / comparison --------------------------------------------
    def short_repr(self) -> str:
        return show_irreps(self.irrep_groups)

    def __repr__(self) -> str:
        return f"Irreps({self.short_repr()})"

    def __hash__(self) -> int:
        return hash(self.short_repr())

    def __eq__(self, other) -> bool:
        if other is None:
            return False
        return self.irrep_groups == check_irreps(other).irrep_groups

    def isomorphic_to(self, other) -> bool:
        return self.simplified() == check_irreps(other).simplified()

    # ---- algebra ---------------------------------------------------------
    def __add__(self, other) -> "Irreps":
        return Irreps(self.irrep_groups + check_irreps(other).irrep_groups)

    def __radd__(self, other) -> "Irreps":
        return Irreps(check_irreps(other).irrep_groups + self.irrep_groups)

    def __mul__(self, other) -> "Irreps":
        other = check_irreps(other)
        acc: List[Tuple[Irrep, int]] = []
        for ir1, m1 in self.irrep_groups:
            for ir2, m2 in other.irrep_groups:
                acc.extend((ir, m1 * m2) for ir in ir1 * ir2)
        return Irreps(acc).simplified()

    def sorted(self, by=None) -> "Irreps":
        """Order by (l, parity None < e < o, multiplicity) unless ``by`` is given."""
        if by is None:
            def by(g):
                return (g[0].l, g[0].p != 0, g[0].p != 1, g[0].p != -1, g[1])
        return Irreps(sorted(self.irrep_groups, key=by))

    def merged(self) -> "Irreps":
        """Fuse adjacent groups of the same irrep."""
        out: List[List] = []
        for ir, mul in self.irrep_groups:
            if out and out[-1][0] == ir:
                out[-1][1] += mul
            else:
                out.append([ir, mul])
        return Irreps([(ir, mul) for ir, mul in out])

    def simplified(self) -> "Irreps":
        """Fuse all groups of the same irrep, then sort."""
        tally: Dict[Irrep, int] = {}
        for ir, mul in self.irrep_groups:
            tally[ir] = tally.get(ir, 0) + mul
        return Irreps(list(tally.items())).sorted()

    def eliminate_parity(self, simplified: bool = False) -> "Irreps":
        out = Irreps([(Irrep(ir.l, 0), mul) for ir, mul in self.irrep_groups])
        return out.simplified() if simplified else out

    # ---- channel bookkeeping ----------------------------------------------
    def channels_divided(self, mul: int) -> "Irreps":
        assert all(m % mul == 0 for _, m in self.irrep_groups), (
            f"All multiplicities must be divisible by {mul}, but got {self.irrep_groups}")
        return Irreps([(ir, m // mul) for ir, m in self.irrep_groups])

    def channels_multiplied(self, mul: int) -> "Irreps":
        return Irreps([(ir, m * mul) for ir, m in self.irrep_groups])

    def max_channels(self) -> int:
        return reduce(math.gcd, (m for _, m in self.irrep_groups))

    def squeeze_max_channels(self) -> Tuple["Irreps", int]:
        g = self.max_channels()
        return self.channels_divided(g), g


def check_irreps(irreps) -> Irreps:
    return irreps if isinstance(irreps, Irreps) else Irreps(irreps)


def has_path(irrep_out: Irrep, irrep_1: Irrep, irrep_2: Irrep = None) -> bool:
    """Selection rule used by the path generators (reference irreps/__init__.py:220-238)."""
    if irrep_2 is None:
        return irrep_out.l == irrep_1.l and (irrep_out.p == 0 or irrep_1.p == irrep_out.p)
    return (abs(irrep_1.l - irrep_2.l) <= irrep_out.l <= irrep_1.l + irrep_2.l
            and (irrep_out.p == 0 or irrep_1.p * irrep_2.p == irrep_out.p))


def unique_irreps(irreps) -> Tuple[Irreps, Dict[Irrep, List[int]]]:
    where: Dict[Irrep, List[int]] = {}
    for pos, ir in enumerate(check_irreps(irreps)):
        where.setdefault(ir, []).append(pos)
    return Irreps(list(where.keys())), where


def irrep_segments(irreps) -> List[int]:
    """Start offset of every (expanded) irrep block plus the total dim."""
    seg = [0]
    for ir in check_irreps(irreps):
        seg.append(seg[-1] + ir.dim)
    return seg


def irrep_indices(irreps) -> torch.Tensor:
    return torch.tensor([i for i, ir in enumerate(check_irreps(irreps)) for _ in range(ir.dim)],
                        dtype=torch.long)


def irrep_degrees(irreps) -> torch.Tensor:
    return torch.tensor([ir.l for ir in check_irreps(irreps)], dtype=torch.long)


def element_degrees(irreps) -> torch.Tensor:
    return torch.tensor([ir.l for ir in check_irreps(irreps) for _ in range(ir.dim)], dtype=torch.long)


def element_orders(irreps) -> torch.Tensor:
    return torch.tensor([m for ir in check_irreps(irreps) for m in range(-ir.l, ir.l + 1)],
                        dtype=torch.long)
