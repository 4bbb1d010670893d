"""Parameter-efficient fine-tuning: low-rank adapters on the decoder's projections and routed experts."""
