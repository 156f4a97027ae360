from torchure_b200.utils.paths import get_project_dir  # noqa: F401
from torchure_b200.utils.segtree import MarkedKeys  # noqa: F401
from torchure_b200.utils.timing import DeviceTimer, debug_time, record_time  # noqa: F401
