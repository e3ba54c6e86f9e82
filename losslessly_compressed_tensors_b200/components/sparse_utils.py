"""Import path of the reference's optimizers (``LCT.components.sparse_utils``)."""
from .optimizers import (  # noqa: F401
    SparseAdamW, SparseMuon, SparseSGDM, muon_update, zeropower_via_newtonschulz5,
)
