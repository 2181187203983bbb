"""Drop-in name for the reference's ``nvfp4_mla.testing`` (nvfp4_mla/testing.py): ``from nvfp4_mla.testing import
RandomCache, SM_SCALE, rel_l2`` is the import form of the reference's tests and benchmarks."""
from nvfp4_mla_b200.testing import *  # noqa: F401,F403
from nvfp4_mla_b200.testing import (CKV, KPE, SM_SCALE, TOKEN_BYTES, RandomCache, SyntheticCache, attention,  # noqa: F401
                                    attention_paged_nvfp4, dequantize, rel_l2)
