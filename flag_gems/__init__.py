"""Drop-in name: ``import flag_gems`` resolves to the B200-native implementation."""
from flaggems_b200 import *  # noqa: F401,F403
from flaggems_b200 import (  # noqa: F401
    __version__,
    _cabi,
    device,
    fused,
    ops,
    patches,
    registration,
    vendor_name,
)
