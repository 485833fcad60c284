"""Model building, the step function, the scheduler and the engine."""
