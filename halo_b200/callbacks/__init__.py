"""Trainer callbacks: efficiency (tokens/s, MFU), MoE load metrics and bias balancing, profiler."""
