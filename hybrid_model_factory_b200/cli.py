"""Console entry point (``hmf`` / ``hybridfactory``): see ``launcher.USAGE``."""
from .launcher import main

if __name__ == "__main__":
    main()
