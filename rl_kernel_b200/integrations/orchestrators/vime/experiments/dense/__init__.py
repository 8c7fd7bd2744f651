"""Dense Qwen3 consistency experiment: a matrix of arms (which module uses the strict operator on which side, whether the
trainer takes the rollout's log-probs), phases (short / precision / convergence / module ablation), one run directory per
arm, validation and collection (parity: rl_engine/integrations/orchestrators/vime/experiments/dense/).

The reference launches the vime orchestrator (Ray + Megatron + vLLM) per arm.  This runtime has its own rollout and
training engines in one process, so an arm is a ``GRPOTrainer`` run; the "framework operator" (P) side of a module is the
library implementation of that module in PyTorch (cuBLAS matmul + log-softmax for the log-prob), which exists for the
log-prob module only -- attention and FFN have no second implementation in this runtime, and arms that ask for one are
reported as unavailable rather than silently run strict."""
