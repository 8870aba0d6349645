"""Per-request history buffers (reference: quickdraw/kvcache/state.py:8-20).

Shapes (reference: quickdraw/engine/engine.py:43-59):
  kv_k, kv_v  bf16 [full_attention_layers, max_context, kv_heads, head_dim]
  rec_state   fp32 [linear_layers, value_heads, key_dim, value_dim]
  conv_state  bf16 [linear_layers, conv_channels, conv_width - 1], oldest tap first
``position`` counts processed tokens; the engine advances it, the step never does.
"""

from dataclasses import dataclass

import torch


@dataclass
class DecodeState:
    kv_k: torch.Tensor
    kv_v: torch.Tensor
    rec_state: torch.Tensor
    conv_state: torch.Tensor
    position: int

    def memory_bytes(self) -> dict[str, int]:
        return {name: getattr(self, name).nbytes
                for name in ("kv_k", "kv_v", "rec_state", "conv_state")}

    @classmethod
    def allocate(cls, config, max_context: int, device) -> "DecodeState":
        full = config.layer_types.count("full_attention")
        linear = config.layer_types.count("linear_attention")
        kv_shape = (full, max_context, config.num_key_value_heads, config.head_dim)
        return cls(
            kv_k=torch.empty(kv_shape, dtype=torch.bfloat16, device=device),
            kv_v=torch.empty(kv_shape, dtype=torch.bfloat16, device=device),
            rec_state=torch.zeros(
                (linear, config.linear_num_value_heads, config.linear_key_head_dim,
                 config.linear_value_head_dim), dtype=torch.float32, device=device),
            conv_state=torch.zeros(
                (linear, config.conv_channels, config.linear_conv_kernel_dim - 1),
                dtype=torch.bfloat16, device=device),
            position=0)
