from .convert_utils import (compress_weight, decompress_weight, reorder_weight,  # noqa: F401
                            transcode_reference_layout, compressed_nbytes)
