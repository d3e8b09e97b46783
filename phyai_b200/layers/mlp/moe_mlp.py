"""Mixture-of-experts MLP: not implemented (the reference ships an empty module at phyai/src/phyai/layers/mlp/moe_mlp.py; the ``ep`` mesh axis exists for it)."""
