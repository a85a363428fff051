"""Drop-in modules for the reference's ffa-fp8fp8 directory."""
