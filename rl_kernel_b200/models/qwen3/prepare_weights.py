"""Materialise and verify a Qwen3 weight snapshot (parity: tools/weights/prepare_ws1_weights.py of the reference).

    python -m rl_kernel_b200.models.qwen3.prepare_weights --output /data/qwen3-8b --verify-only
    python -m rl_kernel_b200.models.qwen3.prepare_weights --output /tmp/tiny --synthetic --layers 2 --hidden 512

``--verify-only`` checks an existing safetensors snapshot: every required tensor present with the model's shapes, shard
checksums against ``--sha256-file`` (a JSON map filename -> sha256) when given, and prints the content hash.  ``--synthetic``
writes a seeded random snapshot of a scaled model in the same layout (for tests and for machines without network access).
Downloading needs ``huggingface_hub`` and a network; it is attempted only when neither flag is given."""
from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

from rl_kernel_b200.models.qwen3 import Qwen3DenseSpec, Qwen3DenseWeights


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--output", type=Path, required=True)
    ap.add_argument("--verify-only", action="store_true")
    ap.add_argument("--synthetic", action="store_true")
    ap.add_argument("--sha256-file", type=Path, default=None)
    ap.add_argument("--seed", type=int, default=0)
    for name, dflt in (("layers", 2), ("hidden", 512), ("ffn", 1536), ("q-heads", 4), ("kv-heads", 2), ("head-dim", 128), ("vocab", 4096)):
        ap.add_argument(f"--{name}", type=int, default=dflt)
    a = ap.parse_args(argv)
    if a.synthetic:
        from safetensors.torch import save_file

        spec = Qwen3DenseSpec.scaled(layers=a.layers, hidden=a.hidden, ffn=a.ffn, q_heads=a.q_heads, kv_heads=a.kv_heads, head_dim=a.head_dim,
                                     vocab=a.vocab)
        w = Qwen3DenseWeights.synthetic(spec, seed=a.seed)
        a.output.mkdir(parents=True, exist_ok=True)
        save_file({f"model.{k}" if k != "lm_head.weight" else k: v.contiguous() for k, v in w.items()}, str(a.output / "model-00001-of-00001.safetensors"))
        (a.output / "spec.json").write_text(json.dumps({"layers": a.layers, "hidden": a.hidden, "ffn": a.ffn, "q_heads": a.q_heads, "kv_heads": a.kv_heads,
                                                        "head_dim": a.head_dim, "vocab": a.vocab, "seed": a.seed}))
    elif not a.verify_only:
        try:
            from huggingface_hub import snapshot_download
        except ImportError as exc:
            print(f"huggingface_hub is required to download weights ({exc}); use --verify-only on a local snapshot", file=sys.stderr)
            return 2
        spec = Qwen3DenseSpec.official()
        a.output.mkdir(parents=True, exist_ok=True)
        snapshot_download(repo_id=spec.model_id, local_dir=a.output, allow_patterns=["model.safetensors.index.json", "model-*.safetensors", "config.json"])
    spec_file = a.output / "spec.json"
    if spec_file.exists():
        s = json.loads(spec_file.read_text())
        spec = Qwen3DenseSpec.scaled(**{k: s[k] for k in ("layers", "hidden", "ffn", "q_heads", "kv_heads", "head_dim", "vocab")})
    else:
        spec = Qwen3DenseSpec.official()
    expected = json.loads(a.sha256_file.read_text()) if a.sha256_file else None
    w = Qwen3DenseWeights.from_hf(spec, a.output, expected_sha256=expected)
    print(json.dumps({"verified": str(a.output), "model": spec.model_id, "tensors": len(list(w.keys())), "content_hash": w.content_hash,
                      "checksums_verified": expected is not None}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
