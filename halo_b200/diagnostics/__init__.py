"""Phase timers on CUDA events, profiler helpers and stack dumps."""
