"""Step function, scheduler and engine loop."""
