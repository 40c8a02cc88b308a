"""Host runtime: KV page manager, batch scheduler, speculator, inferlet processes, messaging."""
