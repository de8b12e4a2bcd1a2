"""Patch-in for the reference's attention backend.

The reference backend module imports two operators and calls one of them per
layer (lazy_attn/lazy/attention/backends/triton_attn.py:13-15, :146-187):
``chunked_prefill_paged_decode`` for the lazy variant and
``chunked_prefill_paged_decode_old`` for the per-token ("mepic") variant.
``install`` rebinds those two names in the backend module to this library's
functions, which accept the same keyword set; ``uninstall`` restores them.
This is the `PatchTarget` pair a maintainer would register in
lazy_attn/lazy/vllm_patch.py:79-110, in a form that also works on an already
imported module.

The operators enqueue their kernels and return, like the reference's; a kernel whose
bounded wait expired (a logic error, never seen in normal operation) can therefore only
report through the device status word.  An engine that installs this patch should call
``lazy_attention_b200.check_device()`` once per step or every few steps: it synchronises,
and raises if any call since the last check produced invalid results.
"""
from __future__ import annotations

import importlib
from types import ModuleType
from typing import Dict, Optional

BACKEND_MODULE = "lazy.attention.backends.triton_attn"
_NAMES = ("chunked_prefill_paged_decode", "chunked_prefill_paged_decode_old")


def install(backend: Optional[ModuleType] = None) -> Dict[str, object]:
    """Rebinds the backend's two operator names; returns the previous bindings."""
    from .attention import chunked_prefill_paged_decode, chunked_prefill_paged_decode_mepic
    if backend is None:
        backend = importlib.import_module(BACKEND_MODULE)
    previous = {n: getattr(backend, n, None) for n in _NAMES}
    backend.chunked_prefill_paged_decode = chunked_prefill_paged_decode
    backend.chunked_prefill_paged_decode_old = chunked_prefill_paged_decode_mepic
    return previous


def uninstall(previous: Dict[str, object], backend: Optional[ModuleType] = None) -> None:
    """Restores the bindings returned by ``install``."""
    if backend is None:
        backend = importlib.import_module(BACKEND_MODULE)
    for n in _NAMES:
        if previous.get(n) is None:
            if hasattr(backend, n):
                delattr(backend, n)
        else:
            setattr(backend, n, previous[n])
