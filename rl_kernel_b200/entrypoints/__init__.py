"""Command-line entry points (``rlk``)."""
