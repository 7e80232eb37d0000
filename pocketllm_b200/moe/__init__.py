"""Mixture-of-experts building blocks: routing, the CPU oracle, model specs / capability /
placement reports, the device MoE layer with expert parallelism."""
