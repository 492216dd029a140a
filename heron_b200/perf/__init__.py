from .perfBuffer import perfBuffer
