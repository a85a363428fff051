"""Drop-in modules for the reference's ffa-nvfp4fp8 directory."""
