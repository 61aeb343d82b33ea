"""flash_mla for B200 (sm_100a): the sparse-MLA path of AppMana/forks-flash-mla-int and its dense sibling.

Same names and argument contract as the reference package (flash_mla/__init__.py:3-15) for
the sparse ops, the int8 row quantizer and dense bf16 paged MLA decode (``get_mla_metadata``,
``flash_mla_with_kvcache``); ``write_fp8_ds_mla_cache`` / ``write_int8_ds_mla_cache``
(encode new rows and scatter them into a paged cache) are additions the reference does not have.  The
int8 dense decoder and the Triton decoder (``flash_mla_with_kvcache_int8``,
``sparse_mla_decode_int8_triton``) are not part of this library.

Importing the package loads the compiled extension; there is no CPU or eager fallback -- a
missing library raises ImportError.
"""
__version__ = "2.0.0+b200"

from .flash_mla_interface import (  # noqa: F401
    flash_mla_with_kvcache,
    get_mla_metadata,
    sparse_mla_decode_fp8,
    sparse_mla_prefill,
)
from .cache_formats import (  # noqa: F401
    int8_ds_mla_cache_views,
    write_fp8_ds_mla_cache,
    write_int8_ds_mla_cache,
)
from .decode_plan import (  # noqa: F401
    SparseMlaDecodePlan,
    device_status_tensor,
    get_sparse_mla_decode_plan,
    sparse_mla_decode_planned,
)
from .int8_sparse_mla import (  # noqa: F401
    quantize_int8_ds_mla_rows,
    sparse_mla_decode_int8,
    sparse_mla_prefill_int8,
)

__all__ = [
    "get_mla_metadata",
    "flash_mla_with_kvcache",
    "sparse_mla_decode_fp8",
    "sparse_mla_prefill",
    "sparse_mla_decode_int8",
    "sparse_mla_prefill_int8",
    "quantize_int8_ds_mla_rows",
    "write_fp8_ds_mla_cache",
    "write_int8_ds_mla_cache",
    "int8_ds_mla_cache_views",
    "get_sparse_mla_decode_plan",
    "sparse_mla_decode_planned",
    "SparseMlaDecodePlan",
    "device_status_tensor",
]
