"""Measurement tools: one kernel or one step at a given size (``probe``), and the larger serving
workloads the benchmark reports beside its headline (``workloads``).  Nothing here is on the
product path."""
