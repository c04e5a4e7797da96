"""Import-only stand-in for the fattorib fused_swiglu package (see compat/README.md)."""
