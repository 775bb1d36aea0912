"""Seeded synthetic workloads with the shapes of the serving benchmarks."""
