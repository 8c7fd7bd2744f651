"""Model families. Qwen3 dense is implemented; the MoE roadmap layer stack lives in ``moe``."""
