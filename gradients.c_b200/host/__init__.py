"""Host-side mirror of the reference interface above the backend ABI."""
