"""The model runner: step function, generation loop, contexts."""
