from .conductor import ConductorPolicy, conductor_policy, resident_prefix
from .loader import BlockSwapLoader, PinnedBlockStore, guard_raw_copy_dtypes
from .plan import BlockPlan, BlockSpec, OffloadConfig, plan_for
from .residency import BudgetTracker, ResidencyManager
from .streamed import StreamedStack
from .telemetry import OffloadTelemetry
