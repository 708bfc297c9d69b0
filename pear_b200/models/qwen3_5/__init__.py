"""The hybrid Gated-DeltaNet + gated-attention model family: recipes, GPU backend selection and the kernel façades the
generic trainer / rollout engine / deploy server install by class path."""
