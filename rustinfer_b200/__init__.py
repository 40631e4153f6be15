"""rustinfer_b200: a small, whole inference engine for decoder-only language models (the Llama-3
dense decoder, the Dirurax hybrid of linear attention and block attention) on one B200 (sm_100a),
with the capabilities RustInfer's decoder path shows."""
from .models import dirurax as _dirurax, linedra as _linedra, llama as _llama, pikalix as _pikalix, sotazen as _sotazen  # noqa: F401  (register the architectures)

__version__ = "0.1.0"
