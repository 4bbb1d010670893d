"""Typed configuration: dataclasses per training method, filled from a YAML file plus
``--key=value`` overrides."""
