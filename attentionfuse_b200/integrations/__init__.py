"""Integrations with downstream libraries (HuggingFace transformers)."""
