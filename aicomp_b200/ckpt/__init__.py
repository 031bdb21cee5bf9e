"""Checkpointing: native per-stage training checkpoints, the HF-compatible stage format and its merge tool."""
