"""Engine: backend contract, step loop, mock / CPU / CUDA backends, exactness harness."""
from .backend import Backend, BackendError, DraftAsk, DraftOffer, RowOutput, RowRequest, TreeRequest  # noqa: F401
from .core import Engine, Event, Request, StepError, TreeConfig, generate  # noqa: F401
from .mock import MockBackend, MockOptions  # noqa: F401
