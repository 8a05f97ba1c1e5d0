"""Host-side mirror of the ChillMask family.

The reference defines a mask as a class whose static functions are inlined into
its Triton kernels (chill_attention/mask.py:15-280).  Here the device side of a
mask is a CUDA functor (csrc/masks.cuh) selected by ``cuda_functor``; this module
keeps the *host* half of the contract with the same names, constructor arguments
and semantics so user code and tests written against the reference keep working:

* ``mask`` / ``k_range_for_q`` / ``q_range_for_k``   (mask.py:54-107)
* ``k_full_range_for_q`` / ``q_full_range_for_k``    (mask.py:109-151)
* ``is_full_block`` / ``has_full_blocks``            (mask.py:212-250)
* ``has_k_full_range`` / ``has_q_full_range`` / ``q_lims_continious`` /
  ``k_lims_continious`` / ``is_guaranteed_safe``     (mask.py:153-210)
* ``make_mask`` / ``make_flex_mask`` / ``verify``    (mask.py:379-534, 700-803)

The static functions work on Python ints and on integer ``torch`` tensors, so the
same definitions serve as documentation, as the CPU tabulation used by
``verify`` and as the expectation the CUDA functors are tested against.
Ranges returned by ``*_range_for_*`` are inclusive, ``*_full_range_for_*`` are
half-open, exactly as in the reference.
"""
from __future__ import annotations

import typing

import torch

_Scalar = typing.Union[int, float, bool]


def _maximum(a, b):
    if isinstance(a, torch.Tensor) or isinstance(b, torch.Tensor):
        return torch.maximum(torch.as_tensor(a), torch.as_tensor(b))
    return max(a, b)


def _minimum(a, b):
    if isinstance(a, torch.Tensor) or isinstance(b, torch.Tensor):
        return torch.minimum(torch.as_tensor(a), torch.as_tensor(b))
    return min(a, b)


def _where(c, a, b):
    if isinstance(c, torch.Tensor):
        return torch.where(c, torch.as_tensor(a), torch.as_tensor(b))
    return a if c else b


def _like(x, value):
    """``value`` broadcast to the shape/type of ``x`` (int stays int)."""
    if isinstance(x, torch.Tensor):
        return torch.zeros_like(x) + value
    return value


def _default_device():
    return "cuda" if torch.cuda.is_available() else "cpu"


class ChillMask:
    """Base class of every attention mask (reference: mask.py:15-52).

    Subclasses pass their constants as a tuple of int/float/bool; ``name`` is the
    class name and is the key under which the dispatcher ops are registered;
    ``str(mask)`` is ``Name(a, b)``.

    Device side: ``cuda_functor`` names the functor struct in csrc/masks.cuh that
    the kernels are instantiated with.  A user-defined mask sets
    ``cuda_functor_header`` to a header that defines a struct of that name with
    the same static member functions; ``register_chill_mask`` then compiles a
    private copy of the kernels for it.
    """

    name: str
    constargs: typing.Tuple[_Scalar, ...]

    #: functor struct name on the CUDA side; ``None`` means "same as class name
    #: without the ChillMask suffix + Mask" for built-ins, required for custom masks
    cuda_functor: typing.Optional[str] = None
    #: path of a user header defining ``cuda_functor`` (custom masks only)
    cuda_functor_header: typing.Optional[str] = None

    def __init__(self, constargs=None):
        self.constargs = constargs or tuple()
        self.name = type(self).__name__
        assert isinstance(self.constargs, tuple), "As of now, only tuple can be passed as args"
        for i in self.constargs:
            assert isinstance(i, (int, float, bool)), (
                "Pytorch interface only supports typing.Union[int, float, bool] parametrization"
            )

    def __str__(self):
        return f"{self.name}({', '.join(map(str, self.constargs))})"

    __repr__ = __str__

    # ------------------------------------------------------------------ contract
    @staticmethod
    def mask(q, k, seq_len, args):
        """bool[m, n]: True where query position q[i] may attend key position k[j]."""
        raise NotImplementedError

    @staticmethod
    def q_range_for_k(k, seq_len, args):
        """Inclusive (first, last) query position that can see key ``k``."""
        raise NotImplementedError

    @staticmethod
    def k_range_for_q(q, seq_len, args):
        """Inclusive (first, last) key position that query ``q`` can see."""
        raise NotImplementedError

    @staticmethod
    def k_full_range_for_q(qb, TILE_Q, seq_len, args):
        """Half-open key range visible to *every* query of the tile [qb, qb+TILE_Q)."""
        return 0, 0

    @staticmethod
    def q_full_range_for_k(kb, TILE_K, seq_len, args):
        """Half-open query range that sees *every* key of the tile [kb, kb+TILE_K)."""
        return 0, 0

    @staticmethod
    def has_k_full_range():
        return False

    @staticmethod
    def has_q_full_range():
        return False

    @staticmethod
    def q_lims_continious():
        return True

    @staticmethod
    def k_lims_continious():
        return True

    @staticmethod
    def is_guaranteed_safe():
        return False

    @staticmethod
    def has_full_blocks(q_tile_size, k_tile_size, seq_len, args):
        return False

    @staticmethod
    def is_full_block(q, k, q_tile_size, k_tile_size, seq_len, args):
        return False

    # ------------------------------------------------------------------- tooling
    def make_mask(self, max_pos, device=None):
        """Dense boolean (max_pos, max_pos) mask, rows = queries (mask.py:379-412)."""
        device = device or _default_device()
        pos = torch.arange(max_pos, device=device, dtype=torch.int64)
        m = type(self).mask(pos, pos, max_pos, self.constargs)
        return torch.as_tensor(m, device=device).expand(max_pos, max_pos).contiguous()

    def _calc_limits(self, max_pos, lim_func, device=None):
        """(max_pos, 2) int32 table of an inclusive range function, clamped to
        max_pos - 1 like the reference's tabulation (mask.py:414-454)."""
        device = device or _default_device()
        pos = torch.arange(max_pos, device=device, dtype=torch.int64)
        lo, hi = lim_func(pos, max_pos, self.constargs)
        lims = torch.stack(
            [torch.as_tensor(lo, device=device).expand(max_pos), torch.as_tensor(hi, device=device).expand(max_pos)],
            dim=1,
        ).to(torch.int32)
        return torch.where(lims >= max_pos, max_pos - 1, lims)

    def _calc_full_block_indices(self, max_pos, q_tile_size, k_tile_size):
        cls = type(self)
        return [
            (q, k)
            for q in range(0, max_pos, q_tile_size)
            for k in range(0, max_pos, k_tile_size)
            if cls.is_full_block(q, k, q_tile_size, k_tile_size, max_pos, self.constargs)
        ]

    def _calc_full_ranges(self, max_pos, tile, rule=None):
        """(n_tiles, 2) int32 table of a half-open full-range function."""
        rule = rule or type(self).k_full_range_for_q
        rows = []
        for i in range(0, max_pos, tile):
            lo, hi = rule(i, tile, max_pos, self.constargs)
            rows.append((int(lo), int(hi)))
        return torch.tensor(rows, dtype=torch.int32).reshape(-1, 2)

    def make_flex_mask(self, max_pos):
        """FlexAttention ``BlockMask`` for the same pattern, or None (mask.py:456-466)."""
        return None

    def mask_mod(self):
        """FlexAttention ``mask_mod(b, h, q_idx, kv_idx)`` callable or None."""
        return None

    def device_tables(self, max_pos, tile, block_tiles=()):
        """Tabulate this mask's CUDA functor on the GPU (the functions the kernels are compiled with, in the library
        ``register_chill_mask`` would use, built on demand for a custom header).  Returns CPU tensors
        ``dense`` bool (n, n), ``k_lims`` / ``q_lims`` int (n, 2), ``k_full`` / ``q_full`` int (ceil(n / tile), 2),
        ``blocks`` {(q_tile, k_tile): bool (n_q_tiles, n_k_tiles)} for the pairs in ``block_tiles`` and ``traits``
        (bit0 has_k_full_range, bit1 has_q_full_range, bit2 k_lims_continious, bit3 q_lims_continious, bit4
        is_guaranteed_safe).  Counterpart of the reference's _mask_infer / _limits_infer / _full_ranges_infer
        (mask.py:284-377, :487-534)."""
        import ctypes

        from . import _cabi
        from .chill import _resolve_functor

        lib, functor_id = _resolve_functor(self)
        n = int(max_pos)
        if not torch.cuda.is_available():
            raise RuntimeError("device tables need a CUDA device")
        dev = torch.device("cuda", torch.cuda.current_device())
        nt = (n + tile - 1) // tile
        dense = torch.empty(n * n, dtype=torch.uint8, device=dev)
        k_lims, q_lims = (torch.empty(n, 2, dtype=torch.int32, device=dev) for _ in range(2))
        k_full, q_full = (torch.empty(nt, 2, dtype=torch.int32, device=dev) for _ in range(2))
        desc = _cabi.mask_desc(functor_id, self.constargs)
        with torch.cuda.device(dev):
            st = _cabi._stream()
            _cabi.check(lib, lib.chill_mask_tabulate(ctypes.byref(desc), n, tile, dense.data_ptr(), k_lims.data_ptr(),
                                                      q_lims.data_ptr(), k_full.data_ptr(), q_full.data_ptr(), st),
                        "chill_mask_tabulate")
            blocks = {}
            for qt, kt in block_tiles:
                full = torch.empty(((n + qt - 1) // qt) * ((n + kt - 1) // kt), dtype=torch.uint8, device=dev)
                _cabi.check(lib, lib.chill_mask_tabulate_blocks(ctypes.byref(desc), n, qt, kt, full.data_ptr(), st),
                            "chill_mask_tabulate_blocks")
                blocks[(qt, kt)] = full
            torch.cuda.synchronize()
        return {
            "dense": dense.cpu().reshape(n, n).bool(), "k_lims": k_lims.cpu().long(), "q_lims": q_lims.cpu().long(),
            "k_full": k_full.cpu().long(), "q_full": q_full.cpu().long(),
            "blocks": {key: v.cpu().reshape((n + key[0] - 1) // key[0], -1).bool() for key, v in blocks.items()},
            "traits": lib.chill_mask_traits(functor_id),
        }

    def verify(self, max_pos, device=False):
        """Consistency check of the whole contract on [0, max_pos)^2.

        Same checks as the reference (mask.py:700-803) - range functions equal
        the true first/last visible position of every row and column,
        ``is_full_block`` never claims a mixed tile, ``k_full_range_for_q`` only
        covers visible keys - plus the one the reference omits:
        ``q_full_range_for_k`` only covers queries that see the whole key tile.

        ``device=False`` checks the Python functions of this class.  ``device=True`` checks the CUDA functor the
        kernels are compiled with (the reference verifies the very functions its kernels inline): the functor is
        tabulated on the GPU (``device_tables``), its mask and range tables must EQUAL this class's Python
        functions, its host predicates must equal the class's, and its own full ranges / ``is_full_block`` must
        hold against its own mask.  A functor whose ``k_range_for_q`` is off by one would silently drop keys in
        the kernels; here it raises.
        """
        cls = type(self)
        if device:
            self._verify_device(max_pos)
            return
        mask = self.make_mask(max_pos, device="cpu")
        assert mask.dtype == torch.bool, "Mask must be boolean"
        n = max_pos
        idx = torch.arange(n)

        def true_limits(m):
            any_ = m.any(dim=1)
            first = torch.where(m, idx[None, :], n).min(dim=1).values
            last = torch.where(m, idx[None, :], -1).max(dim=1).values
            return any_, first, last

        k_lims = self._calc_limits(n, cls.k_range_for_q, device="cpu").long()
        q_lims = self._calc_limits(n, cls.q_range_for_k, device="cpu").long()
        for what, m, lims in (("k lims for q", mask, k_lims), ("q lims for k", mask.t(), q_lims)):
            any_, first, last = true_limits(m)
            bad = any_ & ((first != lims[:, 0]) | (last != lims[:, 1]))
            assert not bad.any(), (
                f"Mismatch real vs analytical {what} at position {int(bad.nonzero()[0])}: "
                f"real=({int(first[bad][0])}, {int(last[bad][0])}) analytical={lims[bad][0].tolist()}"
            )

        for qt in (16, 32, 64, 128, 256):
            for kt in (16, 32, 64, 128, 256):
                if not cls.has_full_blocks(qt, kt, seq_len=n, args=self.constargs):
                    continue
                for q, k in self._calc_full_block_indices(n, qt, kt):
                    tile = mask[q : q + qt, k : k + kt]
                    assert tile.all() or (~tile).all(), (
                        f"is_full_block claims a mixed tile: q={q} k={k} q_tile={qt} k_tile={kt}"
                    )

        if cls.has_k_full_range():
            for tq in (16, 32, 64, 128):
                fr = self._calc_full_ranges(n, tq, cls.k_full_range_for_q)
                for i, (lo, hi) in enumerate(fr.tolist()):
                    qb, qe = i * tq, min(i * tq + tq, n)
                    hi = min(hi, n)
                    if hi > lo:
                        assert mask[qb:qe, lo:hi].all(), (
                            f"k_full_range_for_q [{lo},{hi}) for q tile [{qb},{qe}) has masked pairs"
                        )
        if cls.has_q_full_range():
            for tk in (16, 32, 64, 128):
                fr = self._calc_full_ranges(n, tk, cls.q_full_range_for_k)
                for i, (lo, hi) in enumerate(fr.tolist()):
                    kb, ke = i * tk, min(i * tk + tk, n)
                    hi = min(hi, n)
                    if hi > lo:
                        assert mask[lo:hi, kb:ke].all(), (
                            f"q_full_range_for_k [{lo},{hi}) for k tile [{kb},{ke}) has masked pairs"
                        )

    def _verify_device(self, max_pos):
        cls = type(self)
        n = int(max_pos)
        self.verify(n)  # the Python half first: the device half is compared with it
        py_mask = self.make_mask(n, device="cpu")
        idx = torch.arange(n)
        tiles = (16, 32, 64, 128)
        block_tiles = [(a, b) for a in (16, 64, 128) for b in (16, 64, 128)]
        base = self.device_tables(n, tiles[0], block_tiles)
        dense = base["dense"]
        bad = (dense != py_mask).nonzero()
        assert bad.numel() == 0, (
            f"{self.name}: CUDA functor mask() differs from the Python mask at (q, k) = {tuple(bad[0].tolist())}"
        )
        for what, table, fn in (("k_range_for_q", base["k_lims"], cls.k_range_for_q),
                                ("q_range_for_k", base["q_lims"], cls.q_range_for_k)):
            lo, hi = fn(idx, n, self.constargs)
            exp = torch.stack([torch.as_tensor(lo).expand(n), torch.as_tensor(hi).expand(n)], 1).long()
            # compare where the row / column sees anything at all (an empty range may be written in several ways)
            seen = py_mask.any(dim=1) if what == "k_range_for_q" else py_mask.any(dim=0)
            got = torch.minimum(table, torch.tensor(n - 1))
            exp = torch.minimum(exp, torch.tensor(n - 1))
            bad = (seen[:, None] & (got != exp)).any(dim=1).nonzero()
            assert bad.numel() == 0, (
                f"{self.name}: CUDA functor {what} differs from the Python function at position {int(bad[0])}: "
                f"device {table[int(bad[0])].tolist()} vs python {exp[int(bad[0])].tolist()}"
            )
        tr = base["traits"]
        for bit, fn in ((1, cls.has_k_full_range), (2, cls.has_q_full_range), (4, cls.k_lims_continious),
                        (8, cls.q_lims_continious), (16, cls.is_guaranteed_safe)):
            assert bool(tr & bit) == bool(fn()), f"{self.name}: CUDA functor flag {fn.__name__} = {bool(tr & bit)}, Python says {fn()}"
        for (qt, kt), full in base["blocks"].items():
            for qi, ki in full.nonzero().tolist():
                tile = dense[qi * qt:(qi + 1) * qt, ki * kt:(ki + 1) * kt]
                assert tile.all() or (~tile).all(), (
                    f"{self.name}: CUDA is_full_block claims a mixed tile: q={qi * qt} k={ki * kt} q_tile={qt} k_tile={kt}"
                )
        for t in tiles:
            tab = base if t == tiles[0] else self.device_tables(n, t)
            for name, flag, key in (("k_full_range_for_q", tr & 1, "k_full"), ("q_full_range_for_k", tr & 2, "q_full")):
                if not flag:
                    continue
                for i, (lo, hi) in enumerate(tab[key].tolist()):
                    b, e = i * t, min(i * t + t, n)
                    lo, hi = max(lo, 0), min(hi, n)
                    if hi > lo:
                        sub = dense[b:e, lo:hi] if key == "k_full" else dense[lo:hi, b:e]
                        assert sub.all(), f"{self.name}: CUDA {name} [{lo},{hi}) for tile [{b},{e}) (size {t}) has masked pairs"

    def _flex(self, max_pos):
        from torch.nn.attention.flex_attention import create_block_mask

        return create_block_mask(self.mask_mod(), B=None, H=None, Q_LEN=max_pos, KV_LEN=max_pos)


class FullChillMask(ChillMask):
    """Every query sees every key (reference: mask.py:806-889)."""

    cuda_functor = "FullMask"

    def __init__(self):
        super().__init__()

    @staticmethod
    def mask(q, k, seq_len, args):
        return torch.ones((len(q), len(k)), dtype=torch.bool, device=q.device)

    @staticmethod
    def q_range_for_k(k, seq_len, args):
        return _like(k, 0), _like(k, seq_len - 1)

    @staticmethod
    def k_range_for_q(q, seq_len, args):
        return _like(q, 0), _like(q, seq_len - 1)

    @staticmethod
    def k_full_range_for_q(qb, TILE_Q, seq_len, args):
        return 0, seq_len

    @staticmethod
    def q_full_range_for_k(kb, TILE_K, seq_len, args):
        return 0, seq_len

    @staticmethod
    def has_k_full_range():
        return True

    @staticmethod
    def has_q_full_range():
        return True

    @staticmethod
    def is_guaranteed_safe():
        return True

    @staticmethod
    def has_full_blocks(q_tile_size, k_tile_size, seq_len, args):
        return True

    @staticmethod
    def is_full_block(q, k, q_tile_size, k_tile_size, seq_len, args):
        return True

    def mask_mod(self):
        return lambda b, h, q_idx, kv_idx: q_idx >= 0

    def make_flex_mask(self, max_pos):
        return self._flex(max_pos)


class CausalChillMask(ChillMask):
    """Query q sees keys k <= q (reference: mask.py:892-976)."""

    cuda_functor = "CausalMask"

    def __init__(self):
        super().__init__()

    @staticmethod
    def mask(q, k, seq_len, args):
        return q[:, None] >= k[None, :]

    @staticmethod
    def q_range_for_k(k, seq_len, args):
        return k, _like(k, seq_len - 1)

    @staticmethod
    def k_range_for_q(q, seq_len, args):
        return _like(q, 0), q

    @staticmethod
    def k_full_range_for_q(qb, TILE_Q, seq_len, args):
        return 0, qb + 1

    @staticmethod
    def q_full_range_for_k(kb, TILE_K, seq_len, args):
        return max(0, kb + TILE_K - 1), seq_len

    @staticmethod
    def has_k_full_range():
        return True

    @staticmethod
    def has_q_full_range():
        return True

    @staticmethod
    def is_guaranteed_safe():
        return True

    @staticmethod
    def has_full_blocks(q_tile_size, k_tile_size, seq_len, args):
        return (k_tile_size - 1) <= seq_len - q_tile_size

    @staticmethod
    def is_full_block(q, k, q_tile_size, k_tile_size, seq_len, args):
        return (k + k_tile_size - 1) <= q

    def mask_mod(self):
        return lambda b, h, q_idx, kv_idx: q_idx >= kv_idx

    def make_flex_mask(self, max_pos):
        return self._flex(max_pos)


class SlidingWindowChillMask(ChillMask):
    """Query q sees keys in [q - left_context, q + right_context]
    (reference: mask.py:979-1108)."""

    cuda_functor = "SlidingWindowMask"

    def __init__(self, left_context, right_context):
        super().__init__((left_context, right_context))

    @staticmethod
    def mask(q, k, seq_len, args):
        left, right = args[0], args[1]
        return (k[None, :] <= q[:, None] + right) & (k[None, :] >= q[:, None] - left)

    @staticmethod
    def q_range_for_k(k, seq_len, args):
        left, right = args
        return _maximum(0, k - right), _minimum(k + left, seq_len - 1)

    @staticmethod
    def k_range_for_q(q, seq_len, args):
        left, right = args
        return _maximum(0, q - left), _minimum(q + right, seq_len - 1)

    @staticmethod
    def k_full_range_for_q(qb, TILE_Q, seq_len, args):
        left, right = args
        start = max(0, qb + TILE_Q - 1 - left)
        end = min(seq_len, qb + right + 1)
        return start, max(start, end)

    @staticmethod
    def q_full_range_for_k(kb, TILE_K, seq_len, args):
        # not defined by the reference (it inherits the empty default,
        # mask.py:131-151); same derivation with the roles swapped.
        left, right = args
        start = max(0, kb + TILE_K - 1 - right)
        end = min(seq_len, kb + left + 1)
        return start, max(start, end)

    @staticmethod
    def has_k_full_range():
        return True

    @staticmethod
    def has_q_full_range():
        return True

    @staticmethod
    def is_guaranteed_safe():
        return False

    @staticmethod
    def has_full_blocks(q_tile_size, k_tile_size, seq_len, args):
        left, right = args
        return (
            (q_tile_size <= left and k_tile_size <= right)
            or (q_tile_size * 2 <= left)
            or (k_tile_size * 2 <= right)
        )

    @staticmethod
    def is_full_block(q, k, q_tile_size, k_tile_size, seq_len, args):
        left, right = args[0], args[1]

        def inside(diff):  # diff = q_pos - k_pos of one corner pair
            return (0 <= diff <= left) or (-right <= diff <= 0)

        return inside((q + q_tile_size - 1) - k) and inside(q - (k + k_tile_size - 1))

    def mask_mod(self):
        left, right = self.constargs

        def sliding_window(b, h, q_idx, kv_idx):
            diff = q_idx - kv_idx
            return ((diff <= left) & (diff >= 0)) | ((diff >= -right) & (diff <= 0))

        return sliding_window

    def make_flex_mask(self, max_pos):
        return self._flex(max_pos)


class ChunkwiseChillMask(ChillMask):
    """Sequence cut into chunks of ``context_size``; a query sees its own chunk and
    the ``back_contexts`` chunks before it (reference: mask.py:1111-1266)."""

    cuda_functor = "ChunkwiseMask"

    def __init__(self, context_size, back_contexts):
        super().__init__((context_size, back_contexts))

    @staticmethod
    def mask(q, k, seq_len, args):
        cs, bc = args
        diff = (q // cs)[:, None] - (k // cs)[None, :]
        return (diff >= 0) & (diff <= bc)

    @staticmethod
    def q_range_for_k(k, seq_len, args):
        cs, bc = args
        ck = k // cs
        return ck * cs, _minimum((ck + bc + 1) * cs - 1, seq_len - 1)

    @staticmethod
    def k_range_for_q(q, seq_len, args):
        cs, bc = args
        cq = q // cs
        return _maximum(0, (cq - bc) * cs), _minimum((cq + 1) * cs - 1, seq_len - 1)

    @staticmethod
    def k_full_range_for_q(qb, TILE_Q, seq_len, args):
        cs, bc = args
        start = max(0, ((qb + TILE_Q - 1) // cs - bc) * cs)
        end = min(seq_len, (qb // cs + 1) * cs)
        return start, max(start, end)

    @staticmethod
    def q_full_range_for_k(kb, TILE_K, seq_len, args):
        # not defined by the reference; derived like k_full_range_for_q.
        cs, bc = args
        start = ((kb + TILE_K - 1) // cs) * cs
        end = min(seq_len, (kb // cs + bc + 1) * cs)
        return start, max(start, end)

    @staticmethod
    def has_k_full_range():
        return True

    @staticmethod
    def has_q_full_range():
        return True

    @staticmethod
    def is_guaranteed_safe():
        return False

    @staticmethod
    def has_full_blocks(q_tile_size, k_tile_size, seq_len, args):
        cs, bc = args
        return ChunkwiseChillMask.is_full_block(
            q=cs * (bc + 1) - q_tile_size,
            k=0,
            q_tile_size=q_tile_size,
            k_tile_size=k_tile_size,
            seq_len=seq_len,
            args=args,
        )

    @staticmethod
    def is_full_block(q, k, q_tile_size, k_tile_size, seq_len, args):
        cs, bc = args
        d1 = q // cs - (k + k_tile_size - 1) // cs
        d2 = (q + q_tile_size - 1) // cs - k // cs
        return (0 <= d1 <= bc) and (0 <= d2 <= bc)

    def mask_mod(self):
        cs, bc = self.constargs

        def chunkwise_mask(b, h, q_idx, kv_idx):
            diff = q_idx // cs - kv_idx // cs
            return (diff >= 0) & (diff <= bc)

        return chunkwise_mask

    def make_flex_mask(self, max_pos):
        return self._flex(max_pos)


class PrefixLMChillMask(ChillMask):
    """Keys below ``prefix_size`` are visible to everyone, the rest is causal
    (reference: mask.py:1269-1394)."""

    cuda_functor = "PrefixLMMask"

    def __init__(self, prefix_size):
        super().__init__((prefix_size,))

    @staticmethod
    def mask(q, k, seq_len, args):
        p = args[0]
        return (k < p)[None, :] | (q[:, None] >= k[None, :])

    @staticmethod
    def q_range_for_k(k, seq_len, args):
        p = args[0]
        return _where(k < p, _like(k, 0), k), _like(k, seq_len - 1)

    @staticmethod
    def k_range_for_q(q, seq_len, args):
        p = args[0]
        return _like(q, 0), _minimum(_maximum(q, p - 1), seq_len - 1)

    @staticmethod
    def k_full_range_for_q(qb, TILE_Q, seq_len, args):
        p = args[0]
        return 0, min(max(p, qb + 1), seq_len)

    @staticmethod
    def q_full_range_for_k(kb, TILE_K, seq_len, args):
        # not defined by the reference; a key tile inside the prefix is seen by
        # every query, otherwise the causal rule applies.
        p = args[0]
        if kb + TILE_K <= p:
            return 0, seq_len
        start = max(0, kb + TILE_K - 1)
        return start, max(start, seq_len)

    @staticmethod
    def has_k_full_range():
        return True

    @staticmethod
    def has_q_full_range():
        return True

    @staticmethod
    def is_guaranteed_safe():
        return True

    @staticmethod
    def has_full_blocks(q_tile_size, k_tile_size, seq_len, args):
        return True

    @staticmethod
    def is_full_block(q, k, q_tile_size, k_tile_size, seq_len, args):
        p = args[0]
        return ((k + k_tile_size - 1) <= q) or ((q + q_tile_size <= p) and (k + k_tile_size <= p))

    def mask_mod(self):
        p = self.constargs[0]
        return lambda b, h, q, k: (k < p) | (q >= k)

    def make_flex_mask(self, max_pos):
        return self._flex(max_pos)
