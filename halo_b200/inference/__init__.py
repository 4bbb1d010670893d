"""Clients for served (OpenAI-compatible) endpoints."""
