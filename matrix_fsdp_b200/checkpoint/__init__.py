from ._api import (MatrixStateDictOptions, get_model_state_dict, get_optimizer_state_dict, get_state_dict,
                   matrix_get_state_dict, matrix_set_state_dict, patch_model_state_dict, patch_optimizer_state_dict,
                   set_model_state_dict, set_optimizer_state_dict, set_state_dict)
from .state_dict import (load_matrix_dcp, load_matrix_dcp_full_state, load_matrix_state_dict, matrix_state_dict,
                         read_global_metadata, save_matrix_dcp)
