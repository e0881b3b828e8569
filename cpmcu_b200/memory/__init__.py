from .arena import ALIGN, Arena, PoolExhausted, Region, Workspace, nbytes_of, plan_storage, round_up

__all__ = ["ALIGN", "Arena", "PoolExhausted", "Region", "Workspace", "nbytes_of", "plan_storage", "round_up"]
