"""Package extension point; implementations are registered explicitly."""
