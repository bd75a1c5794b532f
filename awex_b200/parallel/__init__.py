"""Multi-process plumbing: peer memory, flags, process groups."""
