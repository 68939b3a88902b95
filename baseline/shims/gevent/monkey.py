def patch_all(*args, **kwargs):
    pass
