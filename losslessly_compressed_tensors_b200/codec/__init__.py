"""Host-side pipelines of the codec: geometry, encode, decode, fused pointwise updates."""
