"""Drop-in modules for the reference's ffa-fp4fp8 directory."""
