"""Error types of the engine.

One class per failure kind, after the reference's single error enum
(crates/engine/src/error.rs:8-58): shape mismatches, capacity limits, NaN in logits.
(A block table that does not cover its tokens and a page outside the pool are raised by the
native runtime as `RuntimeFault`.)
The loader's errors follow crates/engine/src/weights.rs:66-89.
"""


class EngineError(Exception):
    """Base class of every error the engine raises on purpose."""


class ConfigError(EngineError):
    """config.json is missing a key, has a wrong type or an unsupported value."""


class ShapeError(EngineError):
    """An operand has the wrong shape, dtype, device or alignment for an op."""

    def __init__(self, op: str, msg: str):
        super().__init__(f"{op}: {msg}")
        self.op = op
        self.msg = msg


class CapacityError(EngineError):
    """A request or a batch needs more than a configured limit allows."""

    def __init__(self, what: str, need: int, limit: int):
        super().__init__(f"{what}: need {need}, limit {limit}")
        self.what = what
        self.need = need
        self.limit = limit


class NaNError(EngineError):
    """NaN found where a pick is made from logits (crates/engine/src/backend/cpu/mod.rs:377-379)."""

    def __init__(self, op: str):
        super().__init__(f"{op}: NaN in logits")
        self.op = op


class KernelError(EngineError):
    """A CUDA launch failed, or the kernel library is missing or cannot be built."""


class WeightsError(EngineError):
    """The weights do not fit the model: one error that lists everything wrong."""

    def __init__(self, path, missing=(), unexpected=(), wrong_shape=(), wrong_dtype=(), other=()):
        self.path = str(path)
        self.missing = sorted(missing)
        self.unexpected = sorted(unexpected)
        self.wrong_shape = sorted(wrong_shape)      # (name, expected, actual)
        self.wrong_dtype = sorted(wrong_dtype)      # (name, actual)
        self.other = list(other)
        lines = [f"weights in {self.path} do not fit the model:"]
        if self.missing:
            lines.append(f"  missing ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        for name, exp, act in self.wrong_shape:
            lines.append(f"  wrong shape: {name}: expected {list(exp)}, file has {list(act)}")
        for name, act in self.wrong_dtype:
            lines.append(f"  unsupported dtype: {name}: {act}")
        lines.extend(f"  {o}" for o in self.other)
        super().__init__("\n".join(lines))


class WeightsFormatError(EngineError):
    """The file is not a readable safetensors file."""
