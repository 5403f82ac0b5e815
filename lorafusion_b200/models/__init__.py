"""models sub-package."""
