"""Runtime registry: model manifests, family adapters, execution / shape profiles."""
from .manifest import (ExecutionConfig, ModelManifest, ProductionGuard, ShapeProfile, default_manifest_by_id,  # noqa: F401
                       manifest_for_family, manifest_ids)
from .adapters import Cond, FamilyAdapter, adapter_for, schedule_for  # noqa: F401
