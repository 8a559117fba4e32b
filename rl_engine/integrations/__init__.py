"""Drop-in entry points for other post-training stacks (nothing here imports those stacks at module import)."""
