"""train sub-package."""
