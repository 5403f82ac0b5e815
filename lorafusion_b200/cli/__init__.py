"""cli sub-package."""
