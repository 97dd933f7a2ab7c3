"""Checkpoint and data tools (each module is runnable: python -m savanna_b200.tools.<name> --help)."""
