"""Experiment harnesses (parity: rl_engine/integrations/orchestrators/vime/experiments)."""
