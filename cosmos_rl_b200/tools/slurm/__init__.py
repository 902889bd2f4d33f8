"""SLURM submission helpers (cosmos_rl/tools/slurm/)."""
