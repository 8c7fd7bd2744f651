"""Attention contract (parity: rl_engine/contracts/operators/attention.py:27-1669, reduced to the
schedules this library implements)."""
from __future__ import annotations

import enum
from dataclasses import dataclass, field

from rl_kernel_b200.contracts.operators._base import ContractBase, assert_same_across_ranks

ATTENTION_CONTRACT_ID = "attention.canonical_block128.v1"


class CPLayout(str, enum.Enum):
    NONE = "none"
    CONTIGUOUS = "contiguous"
    ZIGZAG = "zigzag"              # Megatron: rank c owns chunks c and 2cp-1-c
    TOKEN_INTERLEAVED = "token_interleaved"   # rollout prefill-CP pages


class MergeOrder(str, enum.Enum):
    ASCENDING_GLOBAL_BLOCK = "ascending_global_block"


@dataclass(frozen=True)
class ShardingSpec(ContractBase):
    tp_size: int = 1
    cp_size: int = 1
    cp_layout: CPLayout = CPLayout.NONE
    head_parallel: bool = True

    def __post_init__(self):
        for n in (self.tp_size, self.cp_size):
            if n not in (1, 2, 4, 8):
                raise ValueError(f"parallel degrees must be 1, 2, 4 or 8, got {n}")
        if self.tp_size * self.cp_size > 8:
            raise ValueError("tp_size * cp_size must not exceed 8 (one node)")
        if (self.cp_size == 1) != (self.cp_layout == CPLayout.NONE):
            raise ValueError("cp_layout must be NONE exactly when cp_size == 1")


@dataclass(frozen=True)
class ReductionSpec(ContractBase):
    kv_block: int = 128
    merge_order: MergeOrder = MergeOrder.ASCENDING_GLOBAL_BLOCK
    split_kv: bool = False
    accumulate_dtype: str = "float32"
    probability_dtype: str = "bfloat16"
    row_threads: int = 4            # threads that share one query row (fixed: part of the bit contract)

    def __post_init__(self):
        if self.split_kv:
            raise ValueError("split-KV schedules are outside the deterministic contract")
        if self.kv_block != 128:
            raise ValueError("the canonical KV block is 128 keys")


@dataclass(frozen=True)
class KVCacheSpec(ContractBase):
    layout: str = "token_major"     # [seq * max_len, kv_heads * head_dim]
    page_size: int = 128
    dtype: str = "bfloat16"
    zero_initialised: bool = True   # masked keys are multiplied by p = 0, so stale NaNs must not exist


@dataclass(frozen=True)
class RoPESpec(ContractBase):
    theta: float = 1e6
    style: str = "neox_rotate_half"
    table_dtype: str = "float32"
    fused_with_qk_norm: bool = True


@dataclass(frozen=True)
class AttentionProjectionSpec(ContractBase):
    canonical_tp: int = 8
    qkv_layout: str = "gqa_group_major"
    output_tree: str = "balanced_bf16_nodes"


@dataclass(frozen=True)
class AttentionContract(ContractBase):
    num_q_heads: int
    num_kv_heads: int
    head_dim: int = 128
    causal: bool = True
    softmax_scale: float | None = None
    dtype: str = "bfloat16"
    sharding: ShardingSpec = field(default_factory=ShardingSpec)
    reduction: ReductionSpec = field(default_factory=ReductionSpec)
    kv_cache: KVCacheSpec = field(default_factory=KVCacheSpec)
    rope: RoPESpec = field(default_factory=RoPESpec)
    projection: AttentionProjectionSpec = field(default_factory=AttentionProjectionSpec)
    contract_id: str = ATTENTION_CONTRACT_ID

    def __post_init__(self):
        if self.num_q_heads % self.num_kv_heads:
            raise ValueError("q heads must be a multiple of kv heads")
        if self.num_kv_heads % self.sharding.tp_size:
            raise ValueError("tp_size must divide the number of kv heads")
        if not self.causal:
            raise ValueError("only causal attention is contract-bearing")

    def cross_rank_fingerprint(self) -> str:
        """Everything except rank-local fields; equal on all ranks of a correct job."""
        return self.fingerprint()

    def preflight(self, group=None) -> None:
        assert_same_across_ranks(self.cross_rank_fingerprint(), group, "attention contract")


@dataclass(frozen=True)
class AttentionBackendCapability(ContractBase):
    backend_id: str
    head_dims: tuple[int, ...] = (128,)
    dtypes: tuple[str, ...] = ("bfloat16",)
    max_cp: int = 8
    supports_paged_decode: bool = True
    supports_backward: bool = True
    deterministic: bool = True

    def incompatibilities(self, contract: AttentionContract) -> list[str]:
        why = []
        if contract.head_dim not in self.head_dims:
            why.append(f"head_dim {contract.head_dim} not in {self.head_dims}")
        if contract.dtype not in self.dtypes:
            why.append(f"dtype {contract.dtype} not in {self.dtypes}")
        if contract.sharding.cp_size > self.max_cp:
            why.append(f"cp_size {contract.sharding.cp_size} > {self.max_cp}")
        if not self.deterministic:
            why.append("backend is not deterministic")
        return why


B200_ATTENTION_CAPABILITY = AttentionBackendCapability(backend_id="b200-tcgen05")
REFERENCE_ATTENTION_CAPABILITY = AttentionBackendCapability(backend_id="reference", head_dims=(64, 128, 256),
                                                            dtypes=("bfloat16", "float32", "float16"))
