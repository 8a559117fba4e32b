"""Versioned trainer -> rollout weight synchronisation (protocol, transports, engine adapters)."""
