"""Minimal stand-in for the emmy-ml IR package (see ../README.md). Test infrastructure only."""
__version__ = '0.3.11+standin'
