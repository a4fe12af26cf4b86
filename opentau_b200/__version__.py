"""Package version (single source; ``pyproject.toml`` reads the same number)."""

__version__ = "0.1.0"
