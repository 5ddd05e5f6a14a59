"""What every architecture's configuration has in common.

A configuration is a frozen dataclass whose fields are the architecture's own
config.json keys.  `ModelConfig.from_dict` reads them: a key that has no
default must be present, a present key is type-checked, and keys the class does
not know are kept in `extra` (so that writing the configuration back gives the
same file) but never read by model code.
"""
from __future__ import annotations

import dataclasses
import json
from dataclasses import dataclass, field, fields
from pathlib import Path
from typing import Any, ClassVar


class ConfigError(ValueError):
    """A config.json that cannot be used; the message lists every fault found."""


@dataclass(frozen=True)
class ModelConfig:
    """Base of the typed configurations.  Subclasses add the keys of their
    architecture as fields and check them in `validate`."""

    architecture: str = ""
    extra: dict = field(default_factory=dict, compare=False, repr=False)

    # config.json keys that are read but stored under another field name
    _ALIASES: ClassVar[dict[str, str]] = {}

    @classmethod
    def from_dict(cls, d: dict) -> "ModelConfig":
        d = dict(d)
        archs = d.pop("architectures", None)
        arch = d.pop("architecture", None) or (archs[0] if archs else "")
        known = {f.name: f for f in fields(cls) if f.name not in ("architecture", "extra")}
        values: dict[str, Any] = {}
        problems: list[str] = []
        for key in list(d):
            name = cls._ALIASES.get(key, key)
            if name in known:
                values[name] = d.pop(key)
        for name, f in known.items():
            if name not in values:
                if f.default is dataclasses.MISSING and f.default_factory is dataclasses.MISSING:
                    problems.append(f"missing key '{name}'")
                continue
            err = _check_type(name, values[name], f.type)
            if err:
                problems.append(err)
        if problems:
            raise ConfigError(f"{cls.__name__}: " + "; ".join(problems))
        cfg = cls(architecture=arch, extra=d, **values)
        faults = cfg.validate()
        if faults:
            raise ConfigError(f"{cls.__name__}: " + "; ".join(faults))
        return cfg

    @classmethod
    def from_json(cls, path) -> "ModelConfig":
        return cls.from_dict(json.loads(Path(path).read_text()))

    def to_dict(self) -> dict:
        out = {"architectures": [self.architecture]}
        for f in fields(self):
            if f.name in ("architecture", "extra"):
                continue
            out[f.name] = getattr(self, f.name)
        out.update(self.extra)
        return out

    def validate(self) -> list[str]:
        """Faults of the values taken together; empty when the configuration is usable."""
        return []

    # -- what architecture-neutral code asks of any configuration ------------------------
    # Each architecture answers these from its own keys; nothing outside a configuration class
    # reads an architecture's key names.
    @property
    def max_positions(self) -> int | None:
        """The longest sequence the model was made for (None: the configuration sets no limit)."""
        return None

    @property
    def bos_token(self) -> int | None:
        """The token an empty prompt is replaced by (None: the model has none)."""
        return None

    @property
    def stop_tokens(self) -> tuple[int, ...]:
        """Tokens that end a sequence."""
        return ()


_SCALARS = {"int": int, "float": (int, float), "bool": bool, "str": str}


def _check_type(name: str, value: Any, annotation: Any) -> str | None:
    """Checks the plain scalar annotations; others (dicts, unions) are left to `validate`."""
    ann = annotation if isinstance(annotation, str) else getattr(annotation, "__name__", str(annotation))
    want = _SCALARS.get(ann)
    if want is None:
        return None
    if isinstance(value, bool) and want is not bool:
        return f"key '{name}' must be {ann}, got bool"
    if not isinstance(value, want):
        return f"key '{name}' must be {ann}, got {type(value).__name__} ({value!r})"
    return None
