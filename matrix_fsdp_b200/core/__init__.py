from .layout import (LayoutSegment, MatrixGroupLayout, ParamLayout, ParamSegment, RankLayout, ShardPlan,
                     coalesce_segments, contiguous_shard_plan, rank_segments_are_rank_contiguous_chunks)
from .managed_param import ManagedParam, ManagedParamRegistry, ParamRuntimeKind, ParamShardHint
from .mesh import DataParallelMeshDims, DeviceMeshMetadata
from .placement import MatrixShard, MatrixShardPlacement, PlacementCompatibility
from .state import MatrixShardedState
