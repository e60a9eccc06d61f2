"""Federated expert shards: split a MoE checkpoint into a shared part plus one shard per expert,
verify, merge and assemble with overlays (reference: crates/federated/src/shard.rs)."""
from .shard import Manifest, assemble, config_hash, expert_id, merge_to_full, split, split_filtered, verify  # noqa: F401
