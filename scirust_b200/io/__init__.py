from .safetensors import save_safetensors, load_safetensors, serialize, deserialize  # noqa: F401
from .artifacts import (save_weights, load_weights, srt1_to_bytes, srt1_from_bytes, write_manifest,  # noqa: F401
                        parse_manifest, LayerSpec, QModel, QLinear, fnv_bytes, fnv_fold_f32, FNV_INIT)
