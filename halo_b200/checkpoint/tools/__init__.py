"""Offline checkpoint tools: each module has a ``main(argv)`` and runs as ``python -m``."""
