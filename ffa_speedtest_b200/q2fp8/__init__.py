"""Drop-in modules for the reference's ffa-q2fp8 directory."""
