from torchure_b200.data.builder import Collator, build_dataloader, is_synthetic  # noqa: F401
from torchure_b200.data.packers import (BESTFIT_PACKERS, PACKERS, ListPacker, ListPackerBestFit,  # noqa: F401
                                        NumpyPacker, Packer, TensorPacker)
from torchure_b200.data.prefetcher import CUDAPrefetcher  # noqa: F401
from torchure_b200.data.synthetic import SyntheticLoader, synthetic_row  # noqa: F401
