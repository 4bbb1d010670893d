"""Trainer -> rollout weight synchronisation: chunked, bounded, over NVLink peer stores on one box
and over a process-group broadcast otherwise."""
