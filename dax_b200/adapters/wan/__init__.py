from .attn_adapter import DAXWanAttnProcessor2_0, replace_wan_attention
from .functional import optimize_pipe
from .transformer_adapter import quantize_transformer, replace_transformer
from .block_adapter import replace_wan_blocks
