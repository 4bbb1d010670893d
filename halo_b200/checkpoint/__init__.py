"""Checkpoints: standard Hugging Face SafeTensors layouts that ``from_pretrained`` loads, gathered
expert-parallel saves, per-rank optimizer shards with a topology fingerprint, and exact resume."""
