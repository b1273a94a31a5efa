"""Randomised block Hadamard transform along the token axis.

Same surface as the reference's ``HadamardFactory`` / ``HadamardTransform``
(alto/kernels/hadamard_transform/transform.py:15-142): class-level configuration
(``block_size``, ``randomized``, ``dtype``, ``seed``), one shared ``torch.Generator`` from
which the +-1 row-sign vector and then the permutation are drawn, and
``transform(x, left_mul=True) = (W @ x.view(M/n, n, N)) / sqrt(n)`` with
``W = weight[perm][:, perm]``.

The CUDA kernels take the transform as (n, perm, sign): for the Sylvester base matrix
``weight = diag(sign) @ H_n`` (alto/kernels/hadamard_transform/hadamard.py:130-161), so
``y[i] = sign[perm[i]] * (H_n z)[perm[i]]`` with ``z[perm[j]] = x[j]`` and the product by
H_n is an in-register butterfly fused into the quantizers (n = 16).  Every other matrix of size
16, 32 (the reference's default, a table matrix that is not of Sylvester type) or 64 runs through
a dense transform kernel that materialises bf16(H x), as the reference does, followed by a plain
quantizer; other sizes raise.
"""
from __future__ import annotations

from pathlib import Path
from typing import Optional

import torch
from torch import Tensor

from . import _lib as L


def _sylvester(n: int) -> Tensor:
    H = torch.ones(1, 1)
    while H.shape[0] < n:
        H = torch.vstack((torch.hstack((H, H)), torch.hstack((H, -H))))
    return H


def _is_pow2(n: int) -> bool:
    return n > 0 and (n & (n - 1)) == 0


_BASE_CACHE = {}


def _base_matrix(n: int) -> Tensor:
    if n not in _BASE_CACHE:
        _BASE_CACHE[n] = _load_base_matrix(n)
    return _BASE_CACHE[n]


def _load_base_matrix(n: int) -> Tensor:
    """Known Hadamard matrix of size n: the table the reference reads
    (hadamards.safetensors, shipped byte-identically with ``compressed_tensors``) when it is
    installed, else the Sylvester matrix for powers of two."""
    try:
        import compressed_tensors.transform.utils as ctu
        from safetensors import safe_open

        path = Path(ctu.__file__).parent / "hadamards.safetensors"
        with safe_open(str(path), framework="pt", device="cpu") as fh:
            if str(n) in fh.keys():
                return fh.get_tensor(str(n)).float()
    except Exception:  # table not available: only powers of two can be built
        pass
    if not _is_pow2(n):
        raise ValueError(f"Cannot construct random hadamard matrix of size {n}")
    return _sylvester(n)


def deterministic_hadamard_matrix(size: int, dtype=torch.float32, device="cpu") -> Tensor:
    if size <= 0 or not _is_pow2(size):
        raise ValueError("Cannot construct deterministic hadamard of size != 2^n")
    return _sylvester(size).to(dtype=dtype)


def random_hadamard_matrix(size: int, dtype=torch.float32, device="cpu", gen: Optional[torch.Generator] = None):
    """diag(Q) @ H^T with Q drawn as ``torch.randint(0, 2, (size,), dtype=dtype) * 2 - 1``."""
    Q = torch.randint(low=0, high=2, size=(size,), generator=gen, dtype=dtype)
    Q = Q * 2 - 1
    H = _base_matrix(size).to(dtype)
    # The matrix stays on the host: the kernels take it as (perm, sign) launch parameters, and a
    # per-call host-to-device copy would stall the stream on every forward.
    return torch.diag(Q) @ H.t()


class HadamardFactory:
    """Class-level configuration and construction of :class:`HadamardTransform`."""

    block_size: int = 32
    randomized: bool = True
    dtype: torch.dtype = torch.float32
    seed: Optional[int] = None
    generator: torch.Generator = torch.Generator()

    @classmethod
    def configure(cls, block_size: Optional[int] = None, randomized: Optional[bool] = None,
                  dtype: Optional[torch.dtype] = None, seed: Optional[int] = None) -> None:
        if block_size is not None:
            cls.block_size = block_size
        if randomized is not None:
            cls.randomized = randomized
        if dtype is not None:
            cls.dtype = dtype
        if seed is not None:
            cls.seed = seed
            cls.generator.manual_seed(seed)

    @classmethod
    def create_transform(cls, device) -> "HadamardTransform":
        weight = cls._create_weight(device)
        perm = cls._create_permutation(weight) if cls.randomized else None
        return HadamardTransform(weight, perm)

    @classmethod
    def _create_weight(cls, device) -> Tensor:
        if not cls.randomized:
            return deterministic_hadamard_matrix(cls.block_size, cls.dtype, device)
        return random_hadamard_matrix(cls.block_size, cls.dtype, device, cls.generator)

    @classmethod
    def _create_permutation(cls, weight: Tensor) -> Tensor:
        return torch.randperm(weight.size(0), generator=cls.generator)


class HadamardTransform:
    """``weight``: n x n (+-1) matrix; ``perm``: optional permutation applied to its rows and columns."""

    def __init__(self, weight: Tensor, perm: Optional[Tensor]):
        self.weight = weight
        self.perm = perm
        self._scale = torch.tensor(weight.size(0), dtype=torch.float64).sqrt()
        self._rht: Optional[L.Rht] = None
        self._fusable: Optional[bool] = None
        self._dev = {}

    @property
    def n(self) -> int:
        return int(self.weight.size(0))

    def matrix(self) -> Tensor:
        w = self.weight
        if self.perm is not None:
            w = w[self.perm][:, self.perm]
        return w

    @property
    def is_fused(self) -> bool:
        """True when the quantizer kernels can apply the transform themselves: a row-signed
        Sylvester matrix of size 16 (in-register butterfly).  Any other matrix of size 16, 32 or 64
        goes through the dense transform kernel followed by a plain quantizer."""
        if self._fusable is None:
            ok = self.n == 16
            if ok:
                w = self.weight.detach().float().cpu()
                ok = bool(torch.equal(torch.diag(w[:, 0]) @ w, _sylvester(16)))
            self._fusable = ok
        return self._fusable

    def device_params(self) -> L.Rht:
        """(n, perm, sign) for the fused kernels; raises when the transform is not fusable."""
        if self._rht is None:
            if not self.is_fused:
                raise NotImplementedError("this Hadamard matrix is not a row-signed Sylvester matrix of size 16; "
                                          "use the transform itself (dense kernel)")
            n = self.n
            sign = self.weight.detach().float().cpu()[:, 0].clone()
            perm = self.perm.cpu().tolist() if self.perm is not None else list(range(n))
            self._rht = L.Rht(n, perm, [int(v) for v in sign.tolist()])
        return self._rht

    def device_matrix(self, device) -> Tensor:
        """weight[perm][:, perm] as fp32 on ``device`` (uploaded once per transform and device)."""
        key = str(device)
        if key not in self._dev:
            if self.n not in (16, 32, 64):
                raise NotImplementedError(f"Hadamard block sizes 16, 32 and 64 are implemented, got {self.n}")
            self._dev[key] = self.matrix().detach().float().contiguous().to(device)
        return self._dev[key]

    def __call__(self, value: Tensor, inverse: bool = False, left_mul: bool = False) -> Tensor:
        if not value.is_cuda:
            raise RuntimeError("HadamardTransform runs on CUDA tensors only (no CPU fallback)")
        if inverse or not left_mul:
            raise NotImplementedError("only left_mul=True, inverse=False is on the low-precision linear path")
        assert value.dim() == 2, "left_mul expects a [tokens, hidden] matrix"
        torch._check(value.shape[0] % self.n == 0,
                     lambda: f"the token count ({value.shape[0]}) must be a multiple of the Hadamard size {self.n}")
        x = value if (value.stride(1) == 1 and (value.stride(0) * value.element_size()) % 16 == 0) \
            else value.contiguous()
        y = torch.empty_like(x, memory_format=torch.contiguous_format)
        if self.is_fused:
            L.rht_apply(x, y, self.device_params())
        else:
            L.rht_dense(x, y, self.device_matrix(x.device))
        return y
