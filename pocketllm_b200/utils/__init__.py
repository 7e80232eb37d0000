"""Utilities: profiling drivers, roofline arithmetic, logging."""
