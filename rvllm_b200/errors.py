"""Typed errors of the engine.

One base class and one subclass per subsystem, after the reference's single error enum
(v3/crates/rvllm-core/src/error.rs:124-345: Config, Loader, Scheduler, Sampling, Cuda ...).
Errors that can have several causes at once (configuration, weights) carry all of them.
"""
from __future__ import annotations

from typing import List, Sequence


class RvllmError(Exception):
    """Base class of every error the engine raises on purpose."""


class ConfigError(RvllmError):
    """config.json or an engine option is missing, of the wrong type, or inconsistent.

    `reasons` lists every problem found, not only the first
    (v3/crates/rvllm-core/src/config/builder.rs:61-142 accumulates the same way).
    """

    def __init__(self, reasons: Sequence[str] | str, where: str = ""):
        self.reasons: List[str] = [reasons] if isinstance(reasons, str) else list(reasons)
        self.where = where
        head = f"invalid configuration{' in ' + where if where else ''}:"
        super().__init__(head + "".join(f"\n  - {r}" for r in self.reasons))


class LoaderError(RvllmError):
    """A weight file is corrupt, or its tensors do not match the model.

    `missing`, `unexpected` and `wrong_shape` are filled together, so that one error
    shows everything that has to be fixed
    (variants after error.rs:186-214: MissingTensor, ShapeMismatch, DtypeMismatch, Corrupt).
    """

    def __init__(self, message: str = "", *, path: str = "", missing: Sequence[str] = (),
                 unexpected: Sequence[str] = (), wrong_shape: Sequence[str] = (),
                 wrong_dtype: Sequence[str] = ()):
        self.path = path
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)
        self.wrong_dtype = list(wrong_dtype)
        lines = [message or "weights do not match the model"]
        if path:
            lines[0] += f" ({path})"
        for title, items in (("missing tensors", self.missing),
                             ("unexpected tensors", self.unexpected),
                             ("wrong shapes", self.wrong_shape),
                             ("wrong dtypes", self.wrong_dtype)):
            if items:
                lines.append(f"  {title} ({len(items)}):")
                lines.extend(f"    {i}" for i in items)
        super().__init__("\n".join(lines))


class SchedulerError(RvllmError):
    """A request cannot be admitted or scheduled."""


class KvExhausted(SchedulerError):
    """Not enough free cache pages (error.rs:241-245: needed_blocks, free_blocks)."""

    def __init__(self, needed_blocks: int, free_blocks: int, detail: str = ""):
        self.needed_blocks = needed_blocks
        self.free_blocks = free_blocks
        msg = f"cache pages exhausted: need {needed_blocks}, free {free_blocks}"
        super().__init__(msg + (f" ({detail})" if detail else ""))


class SamplingError(RvllmError):
    """Sampling parameters are out of range."""


class KernelError(RvllmError):
    """A CUDA kernel cannot be built, loaded or launched for the sizes it was given."""
