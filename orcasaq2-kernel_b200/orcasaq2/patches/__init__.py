"""Loader patches for engines other than vLLM."""
