// Error convention of the acro:: API: every failed precondition becomes a
// std::runtime_error whose text is "<file>:  <line>  <message>".
// Replaces util/Error.hpp:15-23 of LLNL/acrotensor (same macro name and
// message shape, because user code and tests rely on catching the throw).
#ifndef ACRO_B200_ERROR_HPP
#define ACRO_B200_ERROR_HPP

#include <stdexcept>
#include <string>

namespace acro
{

[[noreturn]] inline void throw_error(const std::string &what)
{
    throw std::runtime_error(what);
}

namespace detail
{
inline std::string located(const char *file, int line, const std::string &msg = std::string())
{
    std::string s(file);
    s += ":  ";
    s += std::to_string(line);
    if (!msg.empty())
    {
        s += "  ";
        s += msg;
    }
    return s;
}
}

#define ACRO_B200_PICK3(a, b, name, ...) name
#define ACROBATIC_ASSERT_BARE(cond) \
    do { if (!(cond)) ::acro::throw_error(::acro::detail::located(__FILE__, __LINE__)); } while (0)
#define ACROBATIC_ASSERT_MSG(cond, msg) \
    do { if (!(cond)) ::acro::throw_error(::acro::detail::located(__FILE__, __LINE__, (msg))); } while (0)
#define ACROBATIC_ASSERT(...) \
    ACRO_B200_PICK3(__VA_ARGS__, ACROBATIC_ASSERT_MSG, ACROBATIC_ASSERT_BARE)(__VA_ARGS__)

}

#endif
