"""Named-dimension shapes over the native ndslice and the mesh-reshaping mixin shared by
ProcMesh, ActorMesh, ValueMesh and DeviceMesh.

Parity: python/monarch/_src/actor/shape.py (MeshTrait: slice/split/flatten/rename/size/
sizes/extent), monarch_hyperactor shape bindings (Shape, Point, Extent).
"""
from __future__ import annotations

from collections.abc import Mapping
from typing import Dict, Iterator, List, Sequence, Tuple, Union

from .. import _native as N

NDSlice = N.Slice
Slice = N.Slice


class Extent:
    """Ordered (label, size) pairs."""

    def __init__(self, labels: Sequence[str], sizes: Sequence[int]):
        if len(labels) != len(sizes):
            raise ValueError("labels and sizes differ in length")
        self._labels = tuple(labels)
        self._sizes = tuple(int(s) for s in sizes)

    @property
    def labels(self) -> Tuple[str, ...]:
        return self._labels

    @property
    def sizes(self) -> Tuple[int, ...]:
        return self._sizes

    @property
    def nelements(self) -> int:
        n = 1
        for s in self._sizes:
            n *= s
        return n

    def __iter__(self) -> Iterator[str]:
        return iter(self._labels)

    def keys(self):
        return self._labels

    def __getitem__(self, label: str) -> int:
        try:
            return self._sizes[self._labels.index(label)]
        except ValueError:
            raise KeyError(label) from None

    def __len__(self) -> int:
        return len(self._labels)

    def __eq__(self, other) -> bool:
        return isinstance(other, Extent) and (self._labels, self._sizes) == (other._labels,
                                                                            other._sizes)

    def __hash__(self) -> int:
        return hash((self._labels, self._sizes))

    def __str__(self) -> str:
        return "{" + ", ".join(f"{l}={s}" for l, s in zip(self._labels, self._sizes)) + "}"

    __repr__ = __str__

    def __reduce__(self):
        return (Extent, (self._labels, self._sizes))


class DimIndexError(IndexError, ValueError):
    """An index outside a dimension (an ``IndexError``; also a ``ValueError``, which is what
    the reference's bindings raise for it)."""


class DimLabelError(KeyError, ValueError):
    """A dimension name the shape does not have (a ``KeyError``; also a ``ValueError``)."""

    def __str__(self) -> str:        # KeyError would show the repr of the message
        return str(self.args[0]) if self.args else ""


class Point(Mapping):
    """A position in an extent: a mapping label -> coordinate with a flat ``rank``."""

    def __init__(self, rank: int, extent: Extent):
        if not 0 <= rank < max(extent.nelements, 1):
            raise ValueError(f"rank {rank} out of range for extent {extent}")
        self._rank = int(rank)
        self._extent = extent

    @property
    def rank(self) -> int:
        return self._rank

    @property
    def extent(self) -> Extent:
        return self._extent

    def size(self, label: str) -> int:
        return self._extent[label]

    def _coords(self) -> Tuple[int, ...]:
        out = []
        r = self._rank
        for s in reversed(self._extent.sizes):
            out.append(r % s)
            r //= s
        return tuple(reversed(out))

    def __getitem__(self, label: str) -> int:
        labels = self._extent.labels
        if label not in labels:
            raise KeyError(label)
        return self._coords()[labels.index(label)]

    def __iter__(self) -> Iterator[str]:
        return iter(self._extent.labels)

    def __len__(self) -> int:
        return len(self._extent.labels)

    def __eq__(self, other) -> bool:
        if isinstance(other, Point):
            return self._rank == other._rank and self._extent == other._extent
        return Mapping.__eq__(self, other)

    def __hash__(self) -> int:
        return hash((self._rank, self._extent))

    def __str__(self) -> str:
        c = self._coords()
        return "{" + ", ".join(f"'{l}': {v}/{s}" for l, v, s in
                               zip(self._extent.labels, c, self._extent.sizes)) + "}"

    __repr__ = __str__

    def __reduce__(self):
        return (Point, (self._rank, self._extent))


class Shape:
    """Labels + a native strided slice of ranks."""

    def __init__(self, labels: Sequence[str], ndslice: N.Slice):
        labels = list(labels)
        if len(labels) != ndslice.ndim:
            raise ValueError(f"{len(labels)} labels for a {ndslice.ndim}-d slice")
        if len(set(labels)) != len(labels):
            raise ValueError(f"duplicate dimension labels in {labels}")
        self._labels = labels
        self._slice = ndslice

    @staticmethod
    def unity() -> "Shape":
        return Shape([], N.Slice(0, [], []))

    @staticmethod
    def row_major(**dims: int) -> "Shape":
        return Shape(list(dims), N.Slice.new_row_major(list(dims.values())))

    @property
    def labels(self) -> List[str]:
        return list(self._labels)

    @property
    def ndslice(self) -> N.Slice:
        return self._slice

    def extent(self) -> Extent:
        return Extent(self._labels, self._slice.sizes)

    def ranks(self) -> List[int]:
        return self._slice.ranks()

    def coordinates(self, rank: int) -> Dict[str, int]:
        return dict(zip(self._labels, self._slice.coordinates(rank)))

    def at(self, label: str, index: int) -> "Shape":
        d = self._dim(label)
        size = self._slice.sizes[d]
        if index < 0:
            index += size
        if not 0 <= index < size:
            raise DimIndexError(f"index {index} out of range for dimension '{label}' of size "
                                f"{size}")
        labels = self._labels[:d] + self._labels[d + 1:]
        return Shape(labels, self._slice.at(d, index))

    def select(self, label: str, sl: slice) -> "Shape":
        d = self._dim(label)
        start, stop, step = sl.indices(self._slice.sizes[d])
        if step <= 0:
            raise ValueError("slice step must be positive")
        return Shape(self._labels, self._slice.select(d, start, max(stop, start), step))

    def index(self, **kwargs: int) -> "Shape":
        s = self
        for k, v in kwargs.items():
            s = s.at(k, v)
        return s

    def _dim(self, label: str) -> int:
        try:
            return self._labels.index(label)
        except ValueError:
            raise DimLabelError(f"{self} does not have dimension {label!r}") from None

    def __len__(self) -> int:
        return len(self._slice)

    def __eq__(self, other) -> bool:
        return isinstance(other, Shape) and self._labels == other._labels and \
            self._slice == other._slice

    def __hash__(self) -> int:
        return hash((tuple(self._labels), self._slice))

    def __str__(self) -> str:
        return "{" + ", ".join(f"{l}={s}" for l, s in zip(self._labels, self._slice.sizes)) + "}"

    def __repr__(self) -> str:
        return f"Shape({self._labels}, {self._slice!r})"

    def __reduce__(self):
        return (Shape, (self._labels, self._slice))


class MeshTrait:
    """Reshaping operations for anything laid out over a :class:`Shape`.

    Implementors provide ``_ndslice``, ``_labels`` and ``_new_with_shape(shape)``; every
    shape handed to ``_new_with_shape`` addresses a subset of the current ranks.
    """

    @property
    def _ndslice(self) -> N.Slice:  # pragma: no cover - interface
        raise NotImplementedError

    @property
    def _labels(self) -> Tuple[str, ...]:  # pragma: no cover - interface
        raise NotImplementedError

    def _new_with_shape(self, shape: Shape):  # pragma: no cover - interface
        raise NotImplementedError

    @property
    def _shape(self) -> Shape:
        own = self.__dict__.get("_shape_value")
        return own if own is not None else Shape(list(self._labels), self._ndslice)

    @_shape.setter
    def _shape(self, shape: Shape) -> None:
        # implementors commonly keep their shape under this very name
        self.__dict__["_shape_value"] = shape

    # -- selection --------------------------------------------------------------------
    def slice(self, **kwargs):
        """``mesh.slice(host=1, gpu=slice(2, 6))``: an int drops the dimension, a slice
        keeps it restricted."""
        shape = self._shape
        for label, v in kwargs.items():
            if isinstance(v, slice):
                shape = shape.select(label, v)
            elif isinstance(v, range):
                shape = shape.select(label, slice(v.start, v.stop, v.step))
            else:
                shape = shape.at(label, int(v))
        return self._new_with_shape(shape)

    # -- reshaping --------------------------------------------------------------------
    def split(self, **kwargs):
        """``mesh.split(host=("dp", "pp"), pp=2)``: existing dims map to tuples of new
        names; new names may carry a size; at most one size per split is inferred."""
        labels = list(self._labels)
        targets: Dict[str, Sequence[str]] = {}
        fixed: Dict[str, int] = {}
        for k, v in kwargs.items():
            if k in labels:
                if isinstance(v, str):
                    raise ValueError(f"expected a sequence of dimensions, but got '{v}'")
                targets[k] = tuple(v)
            else:
                if not isinstance(v, int):
                    raise ValueError(f"'{k}' is not an existing dim. Expected an integer size "
                                     "constraint on a new dim.")
                fixed[k] = v
        sl = self._ndslice
        out_names: List[str] = []
        out_sizes: List[int] = []
        out_strides: List[int] = []
        for name, size, stride in zip(labels, sl.sizes, sl.strides):
            names = targets.get(name, (name,))
            known = 1
            free = None
            for n in names:
                if n in fixed:
                    known *= fixed[n]
                elif free is None:
                    free = n
                else:
                    raise ValueError(f"Cannot infer size of {names} because both {n} and {free} "
                                     f"have unknown size. Specify at least one as argument, "
                                     f"e.g. {n}=4")
            if free is not None:
                q, rem = divmod(size, known)
                if rem:
                    shown = tuple(fixed.get(n, "?") for n in names)
                    raise ValueError(f"Dimension '{name}' of size {size} is not evenly divided by "
                                     f"{names!r} with sizes {shown!r}")
                fixed[free] = q
            elif known != size:
                shown = tuple(fixed[n] for n in names)
                raise ValueError(f"Dimension '{name}' of size {size} is not evenly divided by "
                                 f"{names!r} with sizes {shown!r}")
            sub_sizes = [fixed.pop(n) for n in names]
            st = stride
            sub_strides = []
            for s in reversed(sub_sizes):
                sub_strides.append(st)
                st *= s
            sub_strides.reverse()
            for n in names:
                if n in out_names:
                    raise ValueError(f"Duplicate dimension name '{n}'")
                out_names.append(n)
            out_sizes += sub_sizes
            out_strides += sub_strides
        if fixed:
            raise ValueError(f"unused size constraints: {tuple(fixed.keys())}")
        return self._new_with_shape(Shape(out_names, N.Slice(sl.offset, out_sizes, out_strides)))

    def flatten(self, name: str):
        """All dimensions merged into one (dense meshes only)."""
        sl = self._ndslice
        if not sl.is_contiguous():
            raise ValueError(f"cannot flatten sparse mesh: strides {sl.strides} are not dense "
                             f"for sizes {sl.sizes}")
        return self._new_with_shape(Shape([name], N.Slice(sl.offset, [len(sl)], [1])))

    def rename(self, **kwargs: str):
        return self.split(**{k: (v,) for k, v in kwargs.items()})

    # -- sizes ------------------------------------------------------------------------
    def size(self, dim: Union[None, str, Sequence[str]] = None) -> int:
        if dim is None:
            return len(self._ndslice)
        if isinstance(dim, str):
            if dim not in self._labels:
                raise KeyError(f"{self} does not have dimension {dim!r}")
            return self._ndslice.sizes[list(self._labels).index(dim)]
        n = 1
        for d in dim:
            n *= self.size(d)
        return n

    @property
    def sizes(self) -> Dict[str, int]:
        return dict(zip(self._labels, self._ndslice.sizes))

    @property
    def extent(self) -> Extent:
        return Extent(self._labels, self._ndslice.sizes)

    def __len__(self) -> int:
        return len(self._ndslice)
