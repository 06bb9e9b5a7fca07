from .flashattn_cute import flash_attn_cute, flash_attn_cute_host, flash_attn_status
from .tuner import jit_tuner
