"""Seeded synthetic workloads with the shapes and value distributions of the benchmark
configurations (random-init; no dataset or checkpoint is involved)."""
