"""Command-line entry points (`python -m pocketllm_b200.cli.<name>`)."""
