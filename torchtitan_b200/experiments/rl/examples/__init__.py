"""Worked RL tasks: datasets, environments, reward functions and the configs that tie them to a model."""
