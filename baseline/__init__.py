"""Reference arm of the benchmark: runs the unmodified reference from `baseline/_ref`."""
