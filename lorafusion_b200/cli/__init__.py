"""Command-line drivers; run each as ``python -m lorafusion_b200.cli.<name> --help``."""
