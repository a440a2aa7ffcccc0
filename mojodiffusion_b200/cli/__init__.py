"""Command-line entry points: ``python -m mojodiffusion_b200.cli.sample`` / ``.train`` / ``.train_cadence``."""
