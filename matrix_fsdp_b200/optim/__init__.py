from .flat import FlatShardedAdamW, FlatShardedSGD
from .muon import DEFAULT_MUON_ADJUST_LR_FN, MatrixMuon, newton_schulz_reference
from .state import (LocalOptimizerParamInfo, LocalOptimizerStateTensor, MatrixFSDPOptimizerStateManager,
                    OptimizerStateSummary)
from .wrapper import (ClassifiedMatrixOptimizerParams, MatrixFSDPOptimizer, MatrixOptimizerConfig,
                      MatrixOptimizerParamGroupSummary, MixedMuonAdamWOptimizer, PreparedMatrixOptimizer,
                      classify_matrix_optimizer_params, configure_matrix_optimizer, configure_optimizer,
                      install_matrix_optimizer_auto_prepare, make_mixed_muon_adamw_optimizer,
                      prepare_matrix_optimizer)
