"""B200-native neighbor-list engine behind vesin's C API.

``NeighborList`` mirrors the reference's Python calculator; the compiled
engine lives in ``vesin_b200/lib/libvesin.so`` (built from ``vesin_b200/csrc``
by ``make`` / ``__graft_entry__.build()``).
"""

from ._c_api import LIBRARY_PATH, build_library, get_library  # noqa: F401


def __getattr__(name):
    # torch is only needed by the calculator, not by the build helpers
    if name in ("NeighborList", "set_profiling"):
        from . import _neighbors

        return getattr(_neighbors, name)
    if name in ("BatchNeighborList", "split_batch"):
        from . import _batch

        return getattr(_batch, name)
    if name in ("ShardedNeighborList", "exchange_halo", "owner_of", "choose_axis", "local_set"):
        from . import _sharded

        return getattr(_sharded, name)
    raise AttributeError(name)


__version__ = "0.1.0"
