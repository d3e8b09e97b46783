"""Roofline tooling: a hardware probe, FLOP / byte models of the served models, and per-stage profilers
that put measured stage latencies against them (the counterpart of the reference's ``benchmark/pi05`` and
``benchmark/cosmos3_policy`` folders)."""
