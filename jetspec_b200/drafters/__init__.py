"""Drafters: stubs, draft-head adapters and the oracle-mode benchmark drafter."""
from .base import (Drafter, TreeDrafter, RepeatDrafter, RandomTreeDrafter, TargetEchoDrafter,
                   TargetEchoTreeDrafter)
from .head import DraftHeadDrafter, DraftHeadTreeDrafter, GraphedDraftHead, CompiledDraftHead
from .oracle import OracleTreeDrafter, OracleOverrideDrafter

__all__ = [
    "Drafter", "TreeDrafter", "RepeatDrafter", "RandomTreeDrafter", "TargetEchoDrafter",
    "TargetEchoTreeDrafter", "DraftHeadDrafter", "DraftHeadTreeDrafter", "OracleTreeDrafter",
    "OracleOverrideDrafter", "GraphedDraftHead", "CompiledDraftHead",
]
