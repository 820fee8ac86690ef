"""The error types of the library. Every refusal is an ``InferError`` whose text names what was
refused (as the reference's ``EInferError`` does: ``decoder.pas:3480-3482`` names the
unknown ``model_type``, ``decoder.pas:1937-1949`` the wrong shape)."""


class InferError(Exception):
    """A model, a file, a request or a setting that the library refuses."""


class ConfigError(InferError):
    """config.json is missing a key, has a value out of bounds or asks for what is not built."""


class WeightsError(InferError):
    """The tensors of a model folder do not match what the model binds."""


class CacheError(InferError):
    """A slot or a page was asked for, given back or used in a way the cache refuses."""


class KernelError(InferError):
    """The native library is missing, failed to build, refused a size or reported a fault."""
