"""B200-native provider for the Loom Infer paged-decode hot path.

`api` mirrors the reference's operator interface over the C ABI (include/loom_b200.h);
`build` compiles the CUDA library for sm_100a.  The package has no CPU implementation of the
path: without the built library every entry point raises.
"""
from . import _abi  # noqa: F401
from .api import *  # noqa: F401,F403
from .api import DeviceSpan  # noqa: F401
from .prefill import (Bf16PagedPrefillAlgorithm, Bf16PagedPrefillArgs,  # noqa: F401
                      Bf16PagedPrefillMetadata, Bf16PagedPrefillPlan, Bf16PagedPrefillSpec,
                      PrefillProvider, choose_paged_prefill)
