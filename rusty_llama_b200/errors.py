"""Exception types of the library.

The reference reports every load-time problem as `Error::Format(String)` or
`Error::Io` (src/error.rs:7-12) and never panics on a bad file
(tests/integration.rs:107-120).  The same split is kept here: a bad model
folder raises, it never crashes.
"""


class RustyLlamaError(Exception):
    """Base class of every error this library raises on purpose."""


class ConfigError(RustyLlamaError):
    """config.json is missing a key, has a wrong type, or breaks an invariant."""


class WeightsError(RustyLlamaError):
    """A checkpoint does not match what the model expects.

    `missing`, `unexpected` and `wrong_shape` list every offending tensor, so
    that one failed load tells the whole story.
    """

    def __init__(self, message, missing=(), unexpected=(), wrong_shape=(), wrong_dtype=()):
        super().__init__(message)
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)
        self.wrong_dtype = list(wrong_dtype)


class CacheError(RustyLlamaError):
    """The cache cannot do what was asked: no page or slot left, a slot used
    after it was given back, a slot freed twice."""


class KernelError(RustyLlamaError):
    """A CUDA kernel refused its arguments, could not be built, or the device
    reported an error after its launch."""


class StepError(RustyLlamaError):
    """A batch handed to the step function is not valid (empty, a token id
    outside the vocabulary, an unknown sequence, a position past the limit)."""
