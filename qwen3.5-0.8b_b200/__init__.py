"""B200-native decode path of the Qwen3.5-0.8B text tower: host-side mirror of the
reference engine's step/state/prefill/MTP interface over a C-ABI CUDA library."""
from . import weights  # noqa: F401
from . import build as build_lib  # noqa: F401
from . import engine  # noqa: F401
from . import parallel  # noqa: F401
from . import checkpoint  # noqa: F401
from . import session  # noqa: F401
from . import mtp_adaptive  # noqa: F401
from .engine import Engine, LaneState, MtpRoundGraph, MtpState, Q35Error, StepGraph, load_library  # noqa: F401
