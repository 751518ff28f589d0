from .activations import *
from .deform_conv import *
from .deform_conv_transpose import *
