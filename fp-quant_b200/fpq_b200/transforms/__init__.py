from .transforms import (BaseTransform, HadamardTransform, IdentityTransform, TRANSFORMS, build_transform,
                         get_transform_matrix)
