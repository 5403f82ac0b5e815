"""solver sub-package."""
