"""Import path of the reference's training-side helpers (``swiglu/triton/impls.py``); the names
that have a native counterpart resolve to it, the Triton kernels themselves do not exist here."""
