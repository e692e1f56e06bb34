"""Parts of a decoder. Importing the package registers the standard parts."""
from . import base, plan, standard, latent, experts, recurrent, canon  # noqa: F401
