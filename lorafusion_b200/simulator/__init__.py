"""simulator sub-package."""
