"""Group-relative policy optimisation: advantages, importance ratios and the clipped objective,
token-budget micro-batch planning, rank balancing, and the offline / resident-copy trainers."""
