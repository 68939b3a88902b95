"""Module names of the reference's ``necklace.cuda`` package, mapped onto ``comm`` / ``ops``."""
