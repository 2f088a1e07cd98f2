"""LatticeConfig: the configuration object of the codec API (coset/core/base.py:15-61).

The reference declares a pydantic model whose dataclass-style __post_init__ never runs, so
no field is validated there.  This mirror keeps the same field names and defaults, stays a
plain class (no third-party dependency) and validates only what the CUDA library cannot
represent.  Any object with the attributes q, M, beta and with_dither is accepted by the codec
functions, including the reference's own LatticeConfig.
"""
from typing import Any, Dict


class LatticeConfig:
    _FIELDS = dict(
        lattice_type=None, q=None, M=None, beta=1.0, alpha=1.0, decoding="full",
        check_overload=True, disable_overload_protection=True, disable_scaling=True,
        with_tie_dither=True, with_dither=False, max_scaling_iterations=10,
    )

    def __init__(self, **kwargs):
        unknown = set(kwargs) - set(self._FIELDS)
        if unknown:
            raise TypeError(f"unexpected LatticeConfig fields: {sorted(unknown)}")
        for name, default in self._FIELDS.items():
            if default is None and name not in kwargs:
                raise TypeError(f"LatticeConfig requires '{name}'")
            setattr(self, name, kwargs.get(name, default))
        self.q = int(self.q)
        self.M = int(self.M)
        self.beta = float(self.beta)

    @classmethod
    def from_dict(cls, config_dict: Dict[str, Any]) -> "LatticeConfig":
        return cls(**config_dict)

    def to_dict(self) -> Dict[str, Any]:
        return {name: getattr(self, name) for name in self._FIELDS}

    model_dump = to_dict

    def __repr__(self):
        inner = ", ".join(f"{k}={getattr(self, k)!r}" for k in self._FIELDS)
        return f"LatticeConfig({inner})"

    def __eq__(self, other):
        return isinstance(other, LatticeConfig) and self.to_dict() == other.to_dict()
