"""OmniPlacement: redundant and dynamic expert placement (C++ core in ``csrc/placement``)."""
from .expert_mapping import ExpertMapping, base_pattern, pattern_from_placement  # noqa: F401
from .omni_planner import OmniPlanner  # noqa: F401
