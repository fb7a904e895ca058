"""Launchers and failure injectors: single-box runner/punisher, Slurm helpers, torchx component."""
