"""Selected-token log-prob device operators under the reference's module names."""
