"""B200-native (sm_100a) resident backend for goinfer's ragged batched decode / varlen-prefill step."""
from . import abi, q4k  # noqa: F401
