class BaseTuner:
    """Placeholder for ``isinstance`` checks."""
