"""Headless no-op stand-in for matplotlib: Triton's perf_report plots through pyplot; on a box
without a display or matplotlib the CSV it also writes is the artefact."""
