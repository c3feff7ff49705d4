"""The step function, the scheduler above it and the engine loop."""
