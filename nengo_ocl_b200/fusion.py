"""Fusion of ensemble-pattern operator groups into one kernel per step."""


def fuse_ensemble_groups(sim, groups):
    """Placeholder until the fused kernel is wired in: returns ``groups`` unchanged."""
    return groups


def plan_fused_ensembles(sim, groups):
    raise NotImplementedError
