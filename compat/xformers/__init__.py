"""Import-only stand-in for xformers (see compat/README.md)."""
