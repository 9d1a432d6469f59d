"""The DFlash2 draft on B200: configuration and weights (``weights``), synthetic weights at the checkpoint's scales
(``synthetic``) and the bind-once launch lists of one draft step (``draft``)."""
