"""graph_sampling_b200: B200-native (sm_100a) minibatch graph sampling behind the gSampler (`gs`)
operator surface.  `cabi` binds the C ABI of include/gsb200.h, `ops` mirrors the reference's tensor
operators, `graph.Graph` mirrors gs::Graph, `gs` is the Python face (Matrix, g-SDDMM).  Importing the
package does not need a GPU; creating a context or calling an operator does — there is no CPU path."""
from . import cabi  # noqa: F401

__version__ = "0.1"
