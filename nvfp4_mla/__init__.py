"""Drop-in name: ``import nvfp4_mla`` resolves to the B200 implementation in ``nvfp4_mla_b200``."""
from nvfp4_mla_b200 import *  # noqa: F401,F403
from nvfp4_mla_b200 import __all__, __version__, testing  # noqa: F401
