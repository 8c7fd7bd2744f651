"""Bindings to rollout engines (vLLM-style), trainers (Megatron-style, DeepSpeed) and the vime
orchestrator, plus the weight-sync bridge.  Every binding can be exercised with stand-in framework
classes, so the tests do not need the frameworks installed (parity: rl_engine/integrations)."""
