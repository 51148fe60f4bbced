"""B200-native matmul / batched matmul / Dense path with SwiftRT's operator interface.

Importing the package loads the compiled CUDA library (swiftrt_b200/libsrt_b200.so) and
raises if it has not been built: there is no CPU or PyTorch fallback."""
from ._lib import EXPORTS, SO  # noqa: F401  (raises ImportError when the library is missing)
from .dense import Dense, activation_forward, bias_activation_backward  # noqa: F401
from .matmul import (MatmulError, MatmulOp, check_status, launch_count, matmul, matmul_gradients,  # noqa: F401
                     clear_plan_cache, load_plan_cache, matmul_all_gather_into,
                     matmul_all_gather_multicast_into, matmul_host, matmul_into, query_plan,
                     release_workspaces, save_plan_cache, set_split_k, set_tuning, set_wait_limit, tune)
from .tensor import ActivationType, DataType, Order, empty, order_of  # noqa: F401

KERNEL_SIMT, KERNEL_TCGEN05, KERNEL_TCGEN05_PAIR = 1, 2, 3
from .sharded import shard_range, sharded_matmul, sharded_matmul_host  # noqa: F401,E402
from .peer import PeerBuffer  # noqa: F401,E402
from .recurrent import BasicRNNCell, GRUCell, GraphedSequence, LSTMCell, LSTMState, run_sequence, run_sequence_preconcatenated  # noqa: F401,E402
from .transform import MatrixLayout, leading_dimension, matrix_transform  # noqa: F401,E402
