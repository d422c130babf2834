"""The model, the step function, the scheduler and trace replay."""
