"""Reference-shaped holders of the decode hot path (same names and call signatures as
`iquestrt/kernels/{tail,oproj,router,moe_gemv,ar_tail,prologue}.py`), backed by the C ABI."""

from .ar_tail import MultimemARTail, MultimemMLPTail
from .moe_gemv import MoeDecodeKernels
from .oproj import DenseMlp, OProjGemv
from .prologue import PrologueKernels
from .router import RouterSelect
from .tail import TailKernels

__all__ = ["TailKernels", "OProjGemv", "DenseMlp", "RouterSelect", "MoeDecodeKernels",
           "MultimemARTail", "MultimemMLPTail", "PrologueKernels"]
