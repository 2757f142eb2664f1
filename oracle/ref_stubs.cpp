// Test infrastructure, not product code.
// Definitions for the handful of symbols the reference's training-step objects reference but that live in
// translation units the oracle build leaves out (console parsing needs boost::spirit, the shutdown hook needs
// libsystemd, the orthogonal initializer needs Eigen). None of them is reachable from
// Forward_Pass / Compute__Error / Backward_Pass / Update_Derivative_Weight / Update_Parameter; each aborts if
// it is ever called so that a wrong assumption cannot go unnoticed.
#include "stdafx.hpp"
#include <Strings/String.hpp>
#include <Capturing/Shutdown/Shutdown.hpp>
#include <cstdlib>

void Neural_Network::Initialization__Orthogonal(bool const, T_ const) { std::abort(); }

namespace MyEA::String {
template <typename T> T Cin_Number(T, T, std::string const &) { std::abort(); }
template <typename T> T Cin_Number(T, std::string const &) { std::abort(); }
template <typename T> T Cin_Real_Number(T, T, std::string const &) { std::abort(); }
template <typename T> T Cin_Real_Number(T, std::string const &) { std::abort(); }
template <typename T>
bool Read_Stream_Block_And_Parse_Number(char *&, char *&, size_t &, size_t const, size_t const, T &,
                                        std::vector<char> &, std::ifstream &, char const) { std::abort(); }

template unsigned int Cin_Number<unsigned int>(unsigned int, unsigned int, std::string const &);
template unsigned long Cin_Number<unsigned long>(unsigned long, std::string const &);
template unsigned long Cin_Number<unsigned long>(unsigned long, unsigned long, std::string const &);
template long long Cin_Number<long long>(long long, std::string const &);
template long long Cin_Number<long long>(long long, long long, std::string const &);
template double Cin_Real_Number<double>(double, double, std::string const &);
template double Cin_Real_Number<double>(double, std::string const &);
template float Cin_Real_Number<float>(float, std::string const &);
template float Cin_Real_Number<float>(float, float, std::string const &);
template bool Read_Stream_Block_And_Parse_Number<double>(char *&, char *&, size_t &, size_t const, size_t const,
                                                         double &, std::vector<char> &, std::ifstream &, char const);
template bool Read_Stream_Block_And_Parse_Number<size_t>(char *&, char *&, size_t &, size_t const, size_t const,
                                                         size_t &, std::vector<char> &, std::ifstream &, char const);
void Print_With_Prefix(std::string const &, char const *, ...) {}
bool Accept(std::string const &) { std::abort(); }
std::string To_Upper(std::string text) { return text; }
}  // namespace MyEA::String

namespace MyEA::Capturing { bool Shutdown::Push_Back(std::atomic<bool> *) { return true; } }
