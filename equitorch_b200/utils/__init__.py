"""Host-side helpers: synthetic workloads with the shapes of the benchmark configurations."""
