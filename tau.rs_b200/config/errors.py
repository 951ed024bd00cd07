"""Errors raised while a model folder is read.

The categories follow crates/models/src/error.rs:9-27 (invalid folder, missing file,
invalid configuration, unsupported dtype, unreadable safetensors).
"""


class ModelLoadError(Exception):
    """Base class of every error raised before a model can run."""


class InvalidModelDir(ModelLoadError):
    pass


class MissingFile(ModelLoadError):
    pass


class InvalidConfig(ModelLoadError):
    pass


class UnsupportedDType(ModelLoadError):
    pass


class WeightError(ModelLoadError):
    """Tensors of the folder do not match what the model asks for."""

    def __init__(self, missing, unexpected, wrong_shape, wrong_dtype=()):
        self.missing = sorted(missing)
        self.unexpected = sorted(unexpected)
        self.wrong_shape = sorted(wrong_shape)
        self.wrong_dtype = sorted(wrong_dtype)
        lines = ["model weights do not match the configuration:"]
        if self.missing:
            lines.append(f"  missing tensors ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected tensors ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        for name, found, wanted in self.wrong_shape:
            lines.append(f"  wrong shape: {name} is {list(found)}, expected {list(wanted)}")
        for name, found in self.wrong_dtype:
            lines.append(f"  unsupported storage dtype: {name} is {found}")
        super().__init__("\n".join(lines))


class AllLogitsNaN(RuntimeError):
    """Every logit of a live request's row is NaN: there is nothing to choose from
    (crates/engine/src/generation.rs:81-95 raises the same)."""
